// Host side of the C ABI declared in include/stbpe.h: memory, launches, CUDA graphs.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/stbpe.h"
#include "kernels.cuh"

#define STBPE_VISIBLE __attribute__((visibility("default")))

struct stbpe_engine {
    stbpe_config cfg;
    EngineDev d;
    i64 max_tokens, n_tokens;
    int max_tiles;
    u64 slots;
    Slot *partial;
    i64 *cand;
    u64 lslots;
    int sm_count;
    int merge_grid, count_grid, select_grid, refresh_grid;
    unsigned int merge_slots, count_slots;
    size_t merge_smem, count_smem;
    bool recs_stale, counted;
    bool filter_valid;    // host mirror of DevState::filter_valid
    double filter_density;  // the filter is kept while (matches of the last merge) <= filter_density x tiles
    u64 *dense;           // 65 536 global counters of the byte-level count path
    PartBuffers parts;    // partition buffers of the 16-bit-vocabulary count path (allocated at first use)
    unsigned char *wide_block;             // their allocation: header, fills, hot counters, regions
    u64 *wide_dense;                       // the hot counters inside it
    void *wide_mapped[STBPE_MAX_PEERS];    // peers' allocations as mapped into this process
    WidePeers wide_peers;
    bool wide_open, wide_counted;          // peers mapped / the table holds a count made by stbpe_mg_wide_pass2
    bool full_refresh_pending;             // that count marked no block dirty: the next refresh recomputes all maxima
    i64 dense32_min;      // streams shorter than this use the general kernel
    bool only_bytes;      // every token so far came from stbpe_append_bytes (ids < 256)
    ncclComm_t comm;      // own NCCL communicator for the native multi-GPU round loop
    i64 *all_cands;       // world x 4 gathered candidates (native loop)
    bool own_boxes;
    unsigned char *mail_own;               // this rank's mailbox (peer-memory rounds)
    void *mail_mapped[STBPE_MAX_PEERS];    // peers' mailboxes as mapped into this process
    bool peers_open;
    float count_ms;       // device time of the histogram kernels of the last count
    float convert_ms;     // device time of moving a dense histogram into the pair table (wide path)
    cudaEvent_t ev0, ev1;
    uint32_t *tiles_alt;  // second stream buffer of the re-pack (at creation when memory allows)
    i64 *rp_lens, *rp_offs;  // re-pack scratch: tile lengths and their exclusive sums
    void *rp_tmp;
    size_t rp_tmp_bytes;
    int repacks;
    int repacks_since_load;
    cudaGraphExec_t graph;
    int graph_merges;
    uint32_t *graph_tiles;
    cudaStream_t graph_stream;
    bool use_graph;
    int part_group;       // partitions per launch of the second pass of the partitioned count
    bool use_pdl;         // the captured single-GPU loop launches its kernels as programmatic dependents
    bool pdl_now;         // set while that loop is being captured
    std::string err;
    std::vector<void *> allocs;
};

static thread_local std::string g_create_err;
namespace { struct NcclApi; NcclApi &nccl_api(); void nccl_comm_destroy(void *comm); }

static int fail(stbpe_engine *e, int code, const std::string &msg) {
    if (e)
        e->err = msg;
    else
        g_create_err = msg;
    return code;
}

static int cuda_fail(stbpe_engine *e, cudaError_t c, const char *what) {
    std::string m = std::string(what) + ": " + cudaGetErrorString(c);
    if (c == cudaErrorMemoryAllocation) m = "CUDA out of memory (" + m + ")";
    cudaGetLastError();
    return fail(e, STBPE_E_CUDA, m);
}

#define CK(call)                                                  \
    do {                                                          \
        cudaError_t c_ = (call);                                  \
        if (c_ != cudaSuccess) return cuda_fail(e, c_, #call);    \
    } while (0)

template <typename T>
static cudaError_t dev_alloc(stbpe_engine *e, T **p, size_t count) {
    void *q = nullptr;
    cudaError_t c = cudaMalloc(&q, count * sizeof(T) > 0 ? count * sizeof(T) : 16);
    if (c == cudaSuccess) {
        e->allocs.push_back(q);
        *p = reinterpret_cast<T *>(q);
    }
    return c;
}

static u64 next_pow2(u64 x) {
    u64 p = 1;
    while (p < x) p <<= 1;
    return p;
}

static bool is_device_pointer(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Launch of a loop kernel; with `dependent` and pdl_now set (capture of the single-GPU loop) as a
// programmatic dependent of the kernel before it in the stream: its CTAs may be scheduled once all
// CTAs of that kernel have started, and wait in dep_wait() for it to complete.  Measured on merges
// 8000-10000 of the 1 GiB corpus (61-63 us per merge with plain launches): the worklist and merge
// kernels as dependents save 3.5 us per merge (the merge kernel's shared-memory set-up and CTA
// launch run under the kernels before it); refresh and select as dependents gain nothing, and all
// four together cost 9 us, so only those two are launched this way.
template <typename... Params, typename... Args>
static cudaError_t launch_loop_kernel(const stbpe_engine *e, bool dependent, void (*kernel)(Params...), unsigned int grid,
                                      unsigned int block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (e->pdl_now && dependent) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

extern "C" {

STBPE_VISIBLE const char *stbpe_version(void) { return "stbpe 0.2 (sm_100a)"; }

STBPE_VISIBLE const char *stbpe_last_error(const stbpe_engine *e) {
    return e ? e->err.c_str() : g_create_err.c_str();
}

STBPE_VISIBLE int stbpe_destroy(stbpe_engine *e) {
    if (!e) return STBPE_OK;
    cudaSetDevice(e->cfg.device);
    if (e->graph) cudaGraphExecDestroy(e->graph);
    for (void *&m : e->mail_mapped)
        if (m) {
            cudaIpcCloseMemHandle(m);
            m = nullptr;
        }
    for (void *&m : e->wide_mapped)
        if (m) {
            cudaIpcCloseMemHandle(m);
            m = nullptr;
        }
    // the NCCL communicator is shared by the engines of this process and lives until exit
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    for (void *p : e->allocs) cudaFree(p);
    delete e;
    return STBPE_OK;
}

static int reset_state(stbpe_engine *e, cudaStream_t s) {
    DevState h;
    memset(&h, 0, sizeof(h));
    h.base_vocab = e->cfg.base_vocab;
    CK(cudaMemcpyAsync(e->d.st, &h, sizeof(h), cudaMemcpyHostToDevice, s));
    CK(cudaStreamSynchronize(s));
    e->n_tokens = 0;
    e->d.n_tiles = 0;
    e->recs_stale = true;
    e->counted = false;
    e->only_bytes = true;
    e->filter_valid = false;
    e->wide_counted = e->full_refresh_pending = false;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_create(stbpe_engine **out, const stbpe_config *cfg) {
    if (!out || !cfg) return fail(nullptr, STBPE_E_BADARG, "null argument");
    if (cfg->max_tokens < 0 || cfg->max_merges < 0 || cfg->base_vocab < 0 || cfg->world_size < 1 ||
        cfg->rank < 0 || cfg->rank >= cfg->world_size)
        return fail(nullptr, STBPE_E_BADARG, "invalid configuration");
    if ((i64)cfg->base_vocab + (i64)cfg->max_merges >= 0x7FFFFFFFll)
        return fail(nullptr, STBPE_E_ID_OVERFLOW, "Token id overflow: ids must stay below 2^31-1");
    stbpe_engine *e = new stbpe_engine();
    e->cfg = *cfg;
    e->graph = nullptr;
    e->graph_merges = 0;
    e->tiles_alt = nullptr;
    e->rp_lens = e->rp_offs = nullptr;
    e->rp_tmp = nullptr;
    e->rp_tmp_bytes = 0;
    e->repacks = 0;
    e->repacks_since_load = 0;
    e->count_ms = 0.f;
    e->convert_ms = 0.f;
    e->ev0 = e->ev1 = nullptr;
    e->comm = nullptr;
    e->all_cands = nullptr;
    e->own_boxes = false;
    memset(&e->parts, 0, sizeof(e->parts));
    e->wide_block = nullptr;
    e->wide_dense = nullptr;
    memset(e->wide_mapped, 0, sizeof(e->wide_mapped));
    memset(&e->wide_peers, 0, sizeof(e->wide_peers));
    e->wide_open = e->wide_counted = e->full_refresh_pending = false;
    e->dense32_min = 1ll << 24;
    if (const char *v = getenv("STBPE_DENSE32_MIN_TOKENS")) e->dense32_min = atoll(v);
    e->mail_own = nullptr;
    memset(e->mail_mapped, 0, sizeof(e->mail_mapped));
    e->peers_open = false;
    e->use_graph = getenv("STBPE_NO_GRAPH") == nullptr;
    e->part_group = STBPE_PARTS;
    if (const char *v = getenv("STBPE_PART_GROUP")) e->part_group = atoi(v) > 0 ? atoi(v) : STBPE_PARTS;
    e->use_pdl = getenv("STBPE_NO_PDL") == nullptr;
    e->pdl_now = false;
    e->filter_valid = false;
    e->filter_density = 1.0;
    if (const char *v = getenv("STBPE_FILTER_DENSITY")) e->filter_density = atof(v);
    memset(&e->d, 0, sizeof(e->d));
    auto bail = [&](int code) {
        g_create_err = e->err;
        stbpe_destroy(e);
        return code;
    };
    cudaError_t c = cudaSetDevice(cfg->device);
    if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaSetDevice"));
    cudaDeviceProp prop;
    c = cudaGetDeviceProperties(&prop, cfg->device);
    if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaGetDeviceProperties"));
    e->sm_count = prop.multiProcessorCount;

    e->max_tokens = cfg->max_tokens;
    e->max_tiles = (int)((cfg->max_tokens + STBPE_TILE - 1) / STBPE_TILE);
    if (e->max_tiles < 1) e->max_tiles = 1;
    u64 slots = cfg->table_slots > 0 ? (u64)cfg->table_slots : (u64)cfg->max_tokens / 4;
    if (cfg->table_slots <= 0) {
        // keys are never removed, so the table must hold every pair a run ever creates: 2^27 slots
        // carried 32 000 merges on 2^30 tokens; streams of 2^32 tokens and more get 2^29 (8 GiB)
        const u64 cap = cfg->max_tokens >= (1ll << 32) ? (1ull << 29) : (1ull << 27);
        if (slots < (1ull << 20)) slots = 1ull << 20;
        if (slots > cap) slots = cap;
    }
    slots = next_pow2(slots < (u64)2 * STBPE_PARTS ? (u64)2 * STBPE_PARTS : slots);
    e->slots = slots;
    e->d.mask = slots - 1;
    // table slices: one per partition this rank can own (partitions with its residue modulo the
    // number of ranks), rounded up to a power of two
    u64 slices = next_pow2(((u64)STBPE_PARTS + cfg->world_size - 1) / cfg->world_size);
    e->d.slot_bits = 0;
    while ((slices << e->d.slot_bits) < slots) ++e->d.slot_bits;
    e->d.n_blocks = (unsigned int)(slots / STBPE_BLK);
    e->d.world = cfg->world_size;
    e->d.rank = cfg->rank;

#define ALLOC(ptr, n)                                                  \
    if ((c = dev_alloc(e, &(ptr), (size_t)(n))) != cudaSuccess) return bail(cuda_fail(e, c, "cudaMalloc " #ptr))
    ALLOC(e->d.tiles, (size_t)e->max_tiles * STBPE_TILE);
    ALLOC(e->d.recs, (size_t)e->max_tiles * 2);
    ALLOC(e->d.table, slots);
    ALLOC(e->d.blockmax, e->d.n_blocks);
    ALLOC(e->d.dirty_flag, e->d.n_blocks);
    ALLOC(e->d.dirty_list, e->d.n_blocks);
    e->d.n_super2 = (e->d.n_blocks + 255) / 256;
    ALLOC(e->d.supermax, e->d.n_super2);
    ALLOC(e->d.dirty2_flag, e->d.n_super2);
    ALLOC(e->d.dirty2_list, e->d.n_super2);
    ALLOC(e->d.st, 1);
    ALLOC(e->d.merges, (size_t)2 * (cfg->max_merges + 1));
    ALLOC(e->d.merge_counts, (size_t)cfg->max_merges + 1);
    ALLOC(e->d.live_before, (size_t)cfg->max_merges + 1);
    ALLOC(e->partial, 4096);
    ALLOC(e->dense, 65536);
    ALLOC(e->cand, 4);
    ALLOC(e->all_cands, (size_t)4 * cfg->world_size);
    e->d.presence_words = (unsigned int)(((size_t)e->max_tiles + 31) / 32);
    ALLOC(e->d.presence, (size_t)(STBPE_PROWS + 1) * e->d.presence_words);
    ALLOC(e->d.cand_bits, e->d.presence_words + 1);
    ALLOC(e->d.worklist, (size_t)e->max_tiles + 32);
    // the re-pack allocates nothing inside the merge loop: its scratch is sized here for the largest
    // stream, and the second stream buffer too unless it would take more than half of what is free
    ALLOC(e->rp_lens, (size_t)e->max_tiles + 1);
    ALLOC(e->rp_offs, (size_t)e->max_tiles + 1);
    cub::DeviceScan::ExclusiveSum(nullptr, e->rp_tmp_bytes, e->rp_lens, e->rp_offs, e->max_tiles + 1, 0);
    {
        unsigned char *t = nullptr;
        ALLOC(t, e->rp_tmp_bytes ? e->rp_tmp_bytes : 16);
        e->rp_tmp = t;
    }
    {
        size_t free_b = 0, total_b = 0;
        const size_t want = (size_t)e->max_tiles * STBPE_TILE * sizeof(uint32_t);
        if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess && want <= free_b / 2)
            ALLOC(e->tiles_alt, (size_t)e->max_tiles * STBPE_TILE);
    }
    if (cfg->world_size > 1) {
        e->lslots = 1ull << 22;
        e->d.lmask = e->lslots - 1;
        e->d.cap_per_peer = 0;  // exchange buffers are set by stbpe_mg_set_buffers
        ALLOC(e->d.ltable, e->lslots);
        ALLOC(e->d.ltouched, 2 * e->lslots);
        c = cudaMemset(e->d.ltable, 0xFF, e->lslots * sizeof(Slot));
        if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaMemset ltable"));
        // counts of the local table must start at zero (keys at EMPTY = all ones)
        std::vector<Slot> init(1 << 16);
        for (auto &s : init) { s.key = STBPE_EMPTY; s.count = 0; }
        for (u64 off = 0; off < e->lslots; off += init.size()) {
            c = cudaMemcpy(e->d.ltable + off, init.data(), init.size() * sizeof(Slot), cudaMemcpyHostToDevice);
            if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaMemcpy ltable"));
        }
    }
#undef ALLOC
    c = cudaMemset(e->d.dirty_flag, 0, e->d.n_blocks * sizeof(unsigned int));
    if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaMemset"));
    c = cudaMemset(e->d.dirty2_flag, 0, e->d.n_super2 * sizeof(unsigned int));
    if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaMemset"));

    // launch geometry: persistent CTAs, a whole number per SM
    e->merge_slots = 1024;
    e->count_slots = 8192;
    e->merge_smem = TilePipe::bytes(e->merge_slots);
    e->count_smem = TilePipe::bytes(e->count_slots);
    int occ = 0;
#define SETUP(kern, smem, grid)                                                                         \
    c = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem));           \
    if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaFuncSetAttribute"));                         \
    c = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, STBPE_CTA_THREADS, smem);                      \
    if (c != cudaSuccess) return bail(cuda_fail(e, c, "cudaOccupancyMaxActiveBlocksPerMultiprocessor")); \
    grid = e->sm_count * (occ > 0 ? occ : 1)
    int g1 = 0, g2 = 0;
    SETUP(merge_kernel<false>, e->merge_smem, e->merge_grid);
    SETUP(merge_kernel<true>, e->merge_smem, g1);
    SETUP(count_kernel<false>, e->count_smem, e->count_grid);
    SETUP(count_kernel<true>, e->count_smem, g2);
    if (g1 < e->merge_grid) e->merge_grid = g1;
    if (g2 < e->count_grid) e->count_grid = g2;
#undef SETUP
    e->select_grid = e->sm_count;
    e->refresh_grid = e->sm_count * 4;
    int rc = reset_state(e, 0);
    if (rc != STBPE_OK) return bail(rc);
    *out = e;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_reset(stbpe_engine *e) {
    if (!e) return STBPE_E_BADARG;
    CK(cudaSetDevice(e->cfg.device));
    return reset_state(e, 0);
}

static int append_common(stbpe_engine *e, const void *data, i64 n, size_t elem, const i64 *row_offsets,
                         i64 n_rows, cudaStream_t s) {
    if (n < 0 || n_rows < 0 || (n > 0 && !data)) return fail(e, STBPE_E_BADARG, "bad append arguments");
    if (e->n_tokens + n > e->max_tokens)
        return fail(e, STBPE_E_CAPACITY, "token stream capacity exceeded");
    CK(cudaSetDevice(e->cfg.device));
    if (n == 0) return STBPE_OK;
    if (!e->recs_stale && e->n_tokens > 0) {
        // the stream has been counted: appending is still fine while no merge has rewritten a tile
        // (the tiles are dense and n_tokens is their true length), not afterwards
        DevState h;
        CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
        CK(cudaStreamSynchronize(s));
        if (h.merges_done > 0 || e->repacks_since_load > 0)
            return fail(e, STBPE_E_STATE, "rows cannot be appended after a merge has been applied; call stbpe_reset first");
    }
    uint32_t *dst = e->d.tiles + e->n_tokens;
    unsigned int *bad = &e->d.st->error;
    auto pack = [&](const void *src, i64 cnt, uint32_t *out) {
        if (elem == 1) {
            i64 blocks = (cnt / 16 + 255) / 256 + 1;
            if (blocks > 65535 * 16) blocks = 65535 * 16;
            pack_bytes_kernel<<<(unsigned int)blocks, 256, 0, s>>>((const uint8_t *)src, cnt, out);
        } else {
            i64 blocks = (cnt + 255) / 256;
            if (blocks > 65535 * 16) blocks = 65535 * 16;
            pack_ids_kernel<<<(unsigned int)blocks, 256, 0, s>>>((const int32_t *)src, cnt, out, bad);
        }
    };
    void *staged = nullptr;
    if (is_device_pointer(data)) {
        pack(data, n, dst);
    } else {
        // host data is staged on the device before the pack kernel reads it: in the second stream
        // buffer when the engine has one (it is idle until the first re-pack, and an allocation of this
        // size costs as much as the copy), else in stream-ordered scratch
        char *stage = (char *)e->tiles_alt;
        if (!stage || (size_t)n * elem > (size_t)e->max_tiles * STBPE_TILE * sizeof(uint32_t)) {
            CK(cudaMallocAsync(&staged, (size_t)n * elem, s));
            stage = (char *)staged;
        }
        // the copy goes in pieces on a stream of its own, and every piece is packed on the caller's
        // stream as soon as it has landed, so the pack kernel runs under the following copies
        const i64 piece = (i64)((size_t)(64 << 20) / elem);
        if (n <= piece) {
            CK(cudaMemcpyAsync(stage, data, (size_t)n * elem, cudaMemcpyHostToDevice, s));
            pack(stage, n, dst);
        } else {
            cudaStream_t cs = nullptr;
            cudaEvent_t ready = nullptr, landed = nullptr;
            CK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
            cudaError_t ce = cudaEventCreateWithFlags(&ready, cudaEventDisableTiming);
            if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&landed, cudaEventDisableTiming);
            if (ce == cudaSuccess) ce = cudaEventRecord(ready, s);  // the staging buffer is free once s got here
            if (ce == cudaSuccess) ce = cudaStreamWaitEvent(cs, ready, 0);
            for (i64 at = 0; at < n && ce == cudaSuccess; at += piece) {
                const i64 cnt = n - at < piece ? n - at : piece;
                ce = cudaMemcpyAsync(stage + (size_t)at * elem, (const char *)data + (size_t)at * elem,
                                     (size_t)cnt * elem, cudaMemcpyHostToDevice, cs);
                if (ce == cudaSuccess) ce = cudaEventRecord(landed, cs);
                if (ce == cudaSuccess) ce = cudaStreamWaitEvent(s, landed, 0);  // waits for the record just made
                if (ce == cudaSuccess) pack(stage + (size_t)at * elem, cnt, dst + at);
            }
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(cs);
            if (ready) cudaEventDestroy(ready);
            if (landed) cudaEventDestroy(landed);
            cudaStreamDestroy(cs);
            CK(ce);
        }
    }
    CK(cudaGetLastError());
    // row starts
    std::vector<i64> single = {0, n};
    const i64 *off = row_offsets;
    i64 rows = n_rows;
    if (!off) {
        off = single.data();
        rows = 1;
    } else {
        if (off[0] != 0 || off[rows] != n) {
            if (staged) cudaFreeAsync(staged, s);
            return fail(e, STBPE_E_BADARG, "row_offsets must start at 0 and end at n");
        }
    }
    i64 *doff = nullptr;
    CK(cudaMallocAsync((void **)&doff, (size_t)(rows + 1) * sizeof(i64), s));
    CK(cudaMemcpyAsync(doff, off, (size_t)(rows + 1) * sizeof(i64), cudaMemcpyHostToDevice, s));
    mark_row_starts_kernel<<<(unsigned int)((rows + 255) / 256), 256, 0, s>>>(doff, rows, dst);
    CK(cudaGetLastError());
    CK(cudaFreeAsync(doff, s));
    if (staged) CK(cudaFreeAsync(staged, s));
    // the host offsets (and a host source) must stay valid until the copies ran
    CK(cudaStreamSynchronize(s));
    e->n_tokens += n;
    e->recs_stale = true;
    e->counted = false;
    if (elem != 1) e->only_bytes = false;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_append_bytes(stbpe_engine *e, const uint8_t *data, int64_t n,
                                     const int64_t *row_offsets, int64_t n_rows, void *stream) {
    if (!e) return STBPE_E_BADARG;
    return append_common(e, data, n, 1, (const i64 *)row_offsets, n_rows, (cudaStream_t)stream);
}

STBPE_VISIBLE int stbpe_append_ids(stbpe_engine *e, const int32_t *ids, int64_t n,
                                   const int64_t *row_offsets, int64_t n_rows, void *stream) {
    if (!e) return STBPE_E_BADARG;
    return append_common(e, ids, n, 4, (const i64 *)row_offsets, n_rows, (cudaStream_t)stream);
}

static int check_device_error(stbpe_engine *e, cudaStream_t s) {
    unsigned int err = 0;
    CK(cudaMemcpyAsync(&err, &e->d.st->error, sizeof(err), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    if (err & STBPE_DERR_BAD_ID)
        return fail(e, STBPE_E_ID_OVERFLOW, "Token id overflow: ids must be in [0, 2^31-2]");
    if (err & STBPE_DERR_TABLE_FULL)
        return fail(e, STBPE_E_CAPACITY, "pair workspace capacity exceeded (pair table full: create the engine with more table_slots, GPUBPETrainer.table_slots)");
    if (err & STBPE_DERR_OUTBOX_FULL) return fail(e, STBPE_E_CAPACITY, "pair workspace capacity exceeded (delta outbox full)");
    if (err & STBPE_DERR_LTABLE_FULL) return fail(e, STBPE_E_CAPACITY, "pair workspace capacity exceeded (local delta table full)");
    if (err & STBPE_DERR_TIMEOUT) return fail(e, STBPE_E_TIMEOUT, "a bounded device-side wait gave up (tile pipeline or a peer's flag)");
    if (err & STBPE_DERR_KEY_MISSING) return fail(e, STBPE_E_STATE, "selected pair missing from the pair table");
    return STBPE_OK;
}

static int prepare_stream_state(stbpe_engine *e, cudaStream_t s) {
    if (e->recs_stale) {
        int rc = check_device_error(e, s);  // id range flag from the pack kernels
        if (rc != STBPE_OK) return rc;
        e->d.n_tiles = (int)((e->n_tokens + STBPE_TILE - 1) / STBPE_TILE);
        if (e->d.n_tiles > 0) {
            init_recs_kernel<<<(e->d.n_tiles + 255) / 256, 256, 0, s>>>(e->d, e->n_tokens);
            CK(cudaGetLastError());
        }
        DevState h;
        memset(&h, 0, sizeof(h));
        h.base_vocab = e->cfg.base_vocab;
        h.n_live = e->n_tokens;
        CK(cudaMemcpyAsync(e->d.st, &h, sizeof(h), cudaMemcpyHostToDevice, s));
        CK(cudaStreamSynchronize(s));
        e->recs_stale = false;
        e->repacks_since_load = 0;
        e->filter_valid = false;  // a fresh stream starts without a pair filter (see filter_policy)
    }
    return STBPE_OK;
}

__global__ void clear_skip_state_kernel(EngineDev e, int valid) {
    e.st->n_work = 0;  // a merge that is committed but not yet applied builds its worklist from here
    e.st->filter_valid = valid;
}

// The pair filter follows the tile layout: it is rebuilt from the stream, or declared stale.
static int rebuild_presence(stbpe_engine *e, cudaStream_t s) {
    clear_skip_state_kernel<<<1, 1, 0, s>>>(e->d, 1);
    CK(cudaGetLastError());
    e->filter_valid = true;
    if (e->d.n_tiles > 0) {
        CK(cudaFuncSetAttribute(presence_rebuild_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                STBPE_PROWS * (int)sizeof(unsigned int)));
        presence_rebuild_kernel<<<e->sm_count * 2, 1024, STBPE_PROWS * sizeof(unsigned int), s>>>(e->d);
        CK(cudaGetLastError());
    }
    return STBPE_OK;
}

// Buffers of the partitioned first count (wide_count.cuh), one allocation: every CTA of the first
// pass owns a region of every partition, sized for its share of the partition's words (1 / grid of
// them, give or take the statistics of its batches) plus head room.
static int wide_alloc(stbpe_engine *e) {
    if (e->wide_block) return STBPE_OK;
    const int n_cta = e->sm_count;
    const i64 cap = ((e->max_tokens / STBPE_PARTS / n_cta) * 13 / 10 + 1024 + 3) & ~(i64)3;
    const size_t bytes = STBPE_WIDE_HEADER_BYTES + wide_fill_bytes(n_cta) + 65536 * sizeof(u64) +
                         (size_t)STBPE_PARTS * n_cta * cap * sizeof(uint32_t);
    size_t free_b = 0, total_b = 0;
    CK(cudaMemGetInfo(&free_b, &total_b));
    if (free_b < bytes + ((size_t)2 << 30)) return fail(e, STBPE_E_CAPACITY, "CUDA out of memory (pair partitions)");
    cudaError_t c = dev_alloc(e, &e->wide_block, bytes);
    if (c != cudaSuccess) return cuda_fail(e, c, "cudaMalloc pair partitions");
    WideHeader hd;
    hd.cap = cap;
    hd.n_cta = n_cta;
    CK(cudaMemcpy(e->wide_block, &hd, sizeof(hd), cudaMemcpyHostToDevice));
    e->parts.fill = const_cast<unsigned int *>(wide_fill(e->wide_block));
    e->wide_dense = const_cast<u64 *>(wide_dense(e->wide_block, n_cta));
    e->parts.words = const_cast<uint32_t *>(wide_words(e->wide_block, n_cta));
    e->parts.cap = cap;
    e->parts.n_cta = n_cta;
    return STBPE_OK;
}

// what every count starts with: tile records of a fresh stream, an empty table, no maxima
static int count_prologue(stbpe_engine *e, cudaStream_t s) {
    e->convert_ms = 0.f;
    int rc = prepare_stream_state(e, s);
    if (rc != STBPE_OK) return rc;
    clear_table_kernel<<<e->sm_count * 8, 256, 0, s>>>(e->d);
    CK(cudaGetLastError());
    CK(cudaMemsetAsync(e->d.dirty_flag, 0, e->d.n_blocks * sizeof(unsigned int), s));
    CK(cudaMemsetAsync(e->d.dirty2_flag, 0, e->d.n_super2 * sizeof(unsigned int), s));
    CK(cudaMemsetAsync(e->d.blockmax, 0, (size_t)e->d.n_blocks * sizeof(Slot), s));  // count 0 = no candidate
    CK(cudaMemsetAsync(e->d.supermax, 0, (size_t)e->d.n_super2 * sizeof(Slot), s));
    CK(cudaMemsetAsync(&e->d.st->n_dirty, 0, sizeof(unsigned int), s));
    CK(cudaMemsetAsync(&e->d.st->n_dirty2, 0, sizeof(unsigned int), s));
    CK(cudaMemsetAsync(&e->d.st->n_keys, 0, sizeof(u64), s));
    if (!e->ev0) {
        CK(cudaEventCreate(&e->ev0));
        CK(cudaEventCreate(&e->ev1));
    }
    return STBPE_OK;
}

static bool wide_eligible(const stbpe_engine *e, bool fresh) {
    return e->d.n_tiles > 0 && fresh && !e->only_bytes && e->cfg.base_vocab <= 65536 &&
           e->n_tokens >= e->dense32_min && !getenv("STBPE_NO_DENSE_COUNT");
}

// first pass of the partitioned count; *ok = 0 when an id of 65 536 or more or a full region made it give up
static int wide_pass1(stbpe_engine *e, int *ok, cudaStream_t s) {
    PartBuffers &pb = e->parts;
    *ok = 0;
    CK(cudaMemsetAsync(e->wide_dense, 0, 65536 * sizeof(u64), s));
    CK(cudaEventRecord(e->ev0, s));
    CK(cudaFuncSetAttribute(partition_pairs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STBPE_PART_SMEM_BYTES));
    partition_pairs_kernel<<<pb.n_cta, STBPE_PART_THREADS, STBPE_PART_SMEM_BYTES, s>>>(e->d, e->n_tokens, e->wide_dense, pb);
    CK(cudaGetLastError());
    CK(cudaEventRecord(e->ev1, s));
    unsigned int derr = 0;
    CK(cudaMemcpyAsync(&derr, &e->d.st->error, sizeof(derr), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    CK(cudaEventElapsedTime(&e->count_ms, e->ev0, e->ev1));
    if (derr & STBPE_DERR_DENSE_OVERFLOW) {
        derr &= ~STBPE_DERR_DENSE_OVERFLOW;
        CK(cudaMemcpyAsync(&e->d.st->error, &derr, sizeof(derr), cudaMemcpyHostToDevice, s));
        CK(cudaStreamSynchronize(s));
        return STBPE_OK;
    }
    *ok = 1;
    return STBPE_OK;
}

static int launch_count(stbpe_engine *e, bool mg, cudaStream_t s) {
    if (mg && e->wide_counted) {  // stbpe_mg_wide_pass2 has filled the table already
        e->wide_counted = false;
        return STBPE_OK;
    }
    const bool fresh = e->recs_stale;
    int rc = count_prologue(e, s);
    if (rc != STBPE_OK) return rc;
    if (e->d.n_tiles > 0 && fresh && e->only_bytes && !getenv("STBPE_NO_DENSE_COUNT")) {
        // byte-level fast path: dense stream, ids < 256
        CK(cudaMemsetAsync(e->dense, 0, 65536 * sizeof(u64), s));
        CK(cudaEventRecord(e->ev0, s));
        CK(cudaFuncSetAttribute(count_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4));
        count_dense_kernel<<<e->sm_count, STBPE_DENSE_THREADS, 32768 * 4, s>>>(e->d, e->n_tokens, e->dense);
        CK(cudaGetLastError());
        unsigned int derr = 0;
        CK(cudaMemcpyAsync(&derr, &e->d.st->error, sizeof(derr), cudaMemcpyDeviceToHost, s));
        CK(cudaStreamSynchronize(s));
        if (!(derr & STBPE_DERR_DENSE_OVERFLOW)) {
            if (mg)
                dense_to_table_kernel<true><<<256, 256, 0, s>>>(e->d, e->dense);
            else
                dense_to_table_kernel<false><<<256, 256, 0, s>>>(e->d, e->dense);
            CK(cudaGetLastError());
            CK(cudaEventRecord(e->ev1, s));
            CK(cudaEventSynchronize(e->ev1));
            CK(cudaEventElapsedTime(&e->count_ms, e->ev0, e->ev1));
            return STBPE_OK;
        }
        // a 16-bit counter came too close to its limit: discard and count with the general kernel
        derr &= ~STBPE_DERR_DENSE_OVERFLOW;
        CK(cudaMemcpyAsync(&e->d.st->error, &derr, sizeof(derr), cudaMemcpyHostToDevice, s));
        CK(cudaStreamSynchronize(s));
    }
    if (!mg && wide_eligible(e, fresh)) {
        // 16-bit vocabulary: partition the pairs, then count partition by partition inside L2
        // (wide_count.cuh).  Buffers are allocated at first use and kept for later counts; without
        // room for them the general kernel counts.
        int ok = 0;
        if (wide_alloc(e) == STBPE_OK) {
            rc = wide_pass1(e, &ok, s);
            if (rc != STBPE_OK) return rc;
        }
        if (ok) {
            PartBuffers &pb = e->parts;
            CK(cudaEventRecord(e->ev0, s));
            dense_to_table_kernel<false><<<256, 256, 0, s>>>(e->d, e->wide_dense);
            CK(cudaGetLastError());
            const int per_region = 2;  // blocks per pass-1 region: a region holds some 10^4 words
            // all partitions in a few launches: the blocks of a launch are scheduled in partition
            // order, so two or three table slices are being filled at any time and stay in L2, and
            // the tail of a partition runs under the start of the next
            for (int p = 0; p < STBPE_PARTS; p += e->part_group) {
                const int n = STBPE_PARTS - p < e->part_group ? STBPE_PARTS - p : e->part_group;
                partition_table_kernel<<<pb.n_cta * per_region * n, 1024, 0, s>>>(e->d, pb, p, per_region);
            }
            CK(cudaGetLastError());
            CK(cudaEventRecord(e->ev1, s));
            CK(cudaEventSynchronize(e->ev1));
            CK(cudaEventElapsedTime(&e->convert_ms, e->ev0, e->ev1));
            e->count_ms += e->convert_ms;  // the pair table is complete only after both passes
            return STBPE_OK;
        }
        // an id of 65 536 or more, or a region outgrew its buffer: the general kernel counts
    }
    if (e->d.n_tiles > 0) {
        int grid = e->count_grid < e->d.n_tiles ? e->count_grid : e->d.n_tiles;
        CK(cudaEventRecord(e->ev0, s));
        if (mg)
            count_kernel<true><<<grid, STBPE_CTA_THREADS, e->count_smem, s>>>(e->d, e->count_slots);
        else
            count_kernel<false><<<grid, STBPE_CTA_THREADS, e->count_smem, s>>>(e->d, e->count_slots);
        CK(cudaGetLastError());
        CK(cudaEventRecord(e->ev1, s));
        CK(cudaEventSynchronize(e->ev1));
        CK(cudaEventElapsedTime(&e->count_ms, e->ev0, e->ev1));
    }
    return STBPE_OK;
}

static int launch_refresh(stbpe_engine *e, int all, cudaStream_t s) {
    CK(launch_loop_kernel(e, false, refresh_kernel, e->refresh_grid, 256, 0, s, e->d, all));
    if (all) {  // rebuild the second level as well (a peek changes nothing else)
        CK(cudaMemsetAsync(e->d.dirty2_flag, 0, e->d.n_super2 * sizeof(unsigned int), s));
        select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 0, 1, e->cand);
        CK(cudaGetLastError());
    }
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_count_initial(stbpe_engine *e, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (e->cfg.world_size > 1) return fail(e, STBPE_E_STATE, "use stbpe_mg_count_local on a multi-rank engine");
    int rc = launch_count(e, false, s);
    if (rc != STBPE_OK) return rc;
    rc = launch_refresh(e, 1, s);
    if (rc != STBPE_OK) return rc;
    e->counted = true;
    return check_device_error(e, s);
}

STBPE_VISIBLE int stbpe_select_best(stbpe_engine *e, uint64_t *key, int64_t *count, int64_t *n_ties,
                                    void *stream) {
    if (!e || !key || !count) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (!e->counted) return fail(e, STBPE_E_STATE, "count the pairs before selecting");
    select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 0, 0, e->cand);
    CK(cudaGetLastError());
    if (n_ties) {
        CK(cudaMemsetAsync(&e->d.st->peek_ties, 0, sizeof(i64), s));
        count_ties_kernel<<<e->sm_count * 8, 256, 0, s>>>(e->d);
        CK(cudaGetLastError());
    }
    DevState h;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    *key = h.peek_count > 0 ? h.peek_key : 0;
    *count = h.peek_count;
    if (n_ties) *n_ties = h.peek_count > 0 ? h.peek_ties : 0;
    return STBPE_OK;
}

static int filter_policy(stbpe_engine *e, const DevState &h, bool layout_changed, cudaStream_t s);

static int launch_merge(stbpe_engine *e, bool mg, cudaStream_t s) {
    if (e->d.n_tiles > 0) {
        const int wl_words = (e->d.n_tiles + 31) / 32;
        int wl_grid = (wl_words + 1023) / 1024;
        if (wl_grid > 32) wl_grid = 32;
        CK(launch_loop_kernel(e, true, worklist_kernel, wl_grid, 1024, 0, s, e->d));
        int grid = e->merge_grid < e->d.n_tiles ? e->merge_grid : e->d.n_tiles;
        if (mg)
            CK(launch_loop_kernel(e, true, merge_kernel<true>, grid, STBPE_CTA_THREADS, e->merge_smem, s, e->d, e->merge_slots));
        else
            CK(launch_loop_kernel(e, true, merge_kernel<false>, grid, STBPE_CTA_THREADS, e->merge_smem, s, e->d, e->merge_slots));
    }
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_apply_merge(stbpe_engine *e, int32_t a, int32_t b, int32_t new_id,
                                    int64_t *n_matches, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (!e->counted) return fail(e, STBPE_E_STATE, "count the pairs before merging");
    if (e->cfg.world_size > 1) return fail(e, STBPE_E_STATE, "single-rank entry point");
    if (a < 0 || b < 0 || new_id < 0 || a == 0x7FFFFFFF || b == 0x7FFFFFFF || new_id == 0x7FFFFFFF)
        return fail(e, STBPE_E_ID_OVERFLOW, "Token id overflow: ids must be in [0, 2^31-2]");
    DevState h;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    if (h.merges_done >= e->cfg.max_merges) return fail(e, STBPE_E_CAPACITY, "merge log full");
    force_merge_kernel<<<1, 1, 0, s>>>(e->d, a, b, new_id);
    CK(cudaGetLastError());
    // the count the table held for (a, b) decides whether this merge keeps the pair filter
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    {
        int rc = filter_policy(e, h, false, s);
        if (rc != STBPE_OK) return rc;
    }
    int rc = launch_merge(e, false, s);
    if (rc != STBPE_OK) return rc;
    rc = launch_refresh(e, 0, s);
    if (rc != STBPE_OK) return rc;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    if (n_matches) *n_matches = h.n_matches;
    return check_device_error(e, s);
}

// Keep or drop the pair filter.  A merge whose matches outnumber the tiles visits nearly every tile
// whatever the filter says, while entering its new pairs into the filter costs more than the
// rewrite itself; so the filter is left stale (every merge visits every tile) until the count of the
// last selected pair has fallen to filter_density x tiles, and is then rebuilt from the stream and
// maintained by every later merge.  `h` is the device state as the host has just read it; with
// `layout_changed` the tiles have moved (re-pack), so a filter that is kept must be rebuilt.
static int filter_policy(stbpe_engine *e, const DevState &h, bool layout_changed, cudaStream_t s) {
    if (e->d.n_tiles < 1) return STBPE_OK;
    i64 cnt = h.merges_done > 0 ? h.cur_count : h.peek_count;  // last selected pair, else the best pair of the count
    cnt /= e->cfg.world_size;  // the count is global, the tiles are this rank's
    const bool want = (double)cnt <= e->filter_density * (double)e->d.n_tiles;
    if (want && (!e->filter_valid || layout_changed)) return rebuild_presence(e, s);
    if (layout_changed) {
        clear_skip_state_kernel<<<1, 1, 0, s>>>(e->d, 0);
        CK(cudaGetLastError());
        e->filter_valid = false;
    }
    return STBPE_OK;
}

// Maintenance between batches of merges: dense re-pack of the stream when at most three quarters of
// the tile capacity in use is live, and the pair-filter policy above.  Synchronises the stream.
// *did (may be NULL) tells whether a re-pack happened.
static int maybe_repack(stbpe_engine *e, bool force, int *did, cudaStream_t s) {
    if (did) *did = 0;
    const int nt = e->d.n_tiles;
    if (nt < 1 || e->recs_stale) return STBPE_OK;
    DevState h;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    if (nt < 2 || (!force && (h.n_live * 4 > (i64)nt * STBPE_TILE * 3 || nt < 64)))  // re-pack at <= 75 % fill
        return filter_policy(e, h, false, s);
    if (!e->tiles_alt) CK(dev_alloc(e, &e->tiles_alt, (size_t)e->max_tiles * STBPE_TILE));
    i64 *lens = e->rp_lens, *offs = e->rp_offs;
    CK(cudaMemsetAsync(lens + nt, 0, sizeof(i64), s));
    tile_lens_kernel<<<(nt + 255) / 256, 256, 0, s>>>(e->d, lens);
    CK(cudaGetLastError());
    size_t tmp_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, lens, offs, nt + 1, s);
    if (tmp_bytes > e->rp_tmp_bytes) return fail(e, STBPE_E_STATE, "re-pack scratch too small");
    tmp_bytes = e->rp_tmp_bytes;
    cub::DeviceScan::ExclusiveSum(e->rp_tmp, tmp_bytes, lens, offs, nt + 1, s);
    CK(cudaGetLastError());
    repack_copy_kernel<<<e->sm_count * 8, 256, 0, s>>>(e->d, offs, e->tiles_alt);
    CK(cudaGetLastError());
    i64 total = 0;
    CK(cudaMemcpyAsync(&total, offs + nt, sizeof(i64), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    uint32_t *old = e->d.tiles;
    e->d.tiles = e->tiles_alt;
    e->tiles_alt = old;
    e->d.n_tiles = (int)((total + STBPE_TILE - 1) / STBPE_TILE);
    e->n_tokens = total;  // capacity in use; the merge log keeps the live counts
    if (e->d.n_tiles > 0) {
        init_recs_kernel<<<(e->d.n_tiles + 255) / 256, 256, 0, s>>>(e->d, total);
        CK(cudaGetLastError());
    }
    {
        int rc = filter_policy(e, h, true, s);
        if (rc != STBPE_OK) return rc;
    }
    CK(cudaStreamSynchronize(s));
    e->repacks++;
    e->repacks_since_load++;
    if (did) *did = 1;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_repack(stbpe_engine *e, int force, int *did, void *stream) {
    if (!e) return STBPE_E_BADARG;
    CK(cudaSetDevice(e->cfg.device));
    return maybe_repack(e, force != 0, did, (cudaStream_t)stream);
}

__global__ void set_target_kernel(EngineDev e, int target) {
    e.st->target = target;
    e.st->stopped = 0;
    e.st->stop_reason = 0;
    e.st->n_matches = 0;
}

// One iteration of the single-GPU loop: select, worklist, merge, refresh.  (Folding refresh, select
// and the worklist into one launch was tried: the CTA that finishes last then recomputes the dirty
// super-block maxima and walks the filter rows alone, and since early in a run nearly every
// super-block is dirty that took 85-400 us per merge instead of the 30 us of the three launches.)
static int enqueue_iteration(stbpe_engine *e, cudaStream_t s) {
    CK(launch_loop_kernel(e, false, select_kernel, e->select_grid, STBPE_SELECT_THREADS, 0, s, e->d, 1, 0, e->cand, 0));
    int rc = launch_merge(e, false, s);
    if (rc != STBPE_OK) return rc;
    return launch_refresh(e, 0, s);
}

STBPE_VISIBLE int stbpe_train(stbpe_engine *e, int32_t n_merges, void *stream) {
    if (!e || n_merges < 0) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (!e->counted) return fail(e, STBPE_E_STATE, "count the pairs before training");
    if (e->cfg.world_size > 1) return fail(e, STBPE_E_STATE, "single-rank entry point");
    DevState h;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    i64 target = (i64)h.merges_done + n_merges;
    if (target > e->cfg.max_merges) target = e->cfg.max_merges;
    set_target_kernel<<<1, 1, 0, s>>>(e->d, (int)target);
    CK(cudaGetLastError());
    int todo = (int)(target - h.merges_done);
    const int G = 32, CHECK = 256;  // merges per graph replay / per look at the device state
    while (todo > 0) {
        int rc = maybe_repack(e, false, nullptr, s);
        if (rc != STBPE_OK) return rc;
        // while the pair filter is stale the counts are looked at after every graph replay, so that
        // tile skipping starts soon after it begins to pay
        const int chk = (e->filter_valid || e->d.n_tiles < 64) ? CHECK : G;
        int batch = todo < chk ? todo : chk;
        todo -= batch;
        if (e->use_graph && batch >= G) {
            // the kernels take all their work from device state, so one captured batch of G
            // iterations is replayed; iterations past a stop rule return immediately
            if (e->graph && (e->graph_merges != e->d.n_tiles || e->graph_tiles != e->d.tiles)) {
                cudaGraphExecDestroy(e->graph);
                e->graph = nullptr;
            }
            if (!e->graph) {
                cudaStream_t cs;
                CK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
                cudaGraph_t g;
                CK(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal));
                int rc2 = STBPE_OK;
                e->pdl_now = e->use_pdl;
                for (int i = 0; i < G && rc2 == STBPE_OK; ++i) rc2 = enqueue_iteration(e, cs);
                e->pdl_now = false;
                cudaError_t ce = cudaStreamEndCapture(cs, &g);
                if (rc2 != STBPE_OK) {
                    cudaStreamDestroy(cs);
                    return rc2;
                }
                if (ce != cudaSuccess) {
                    cudaStreamDestroy(cs);
                    return cuda_fail(e, ce, "cudaStreamEndCapture");
                }
                ce = cudaGraphInstantiate(&e->graph, g, 0);
                cudaGraphDestroy(g);
                cudaStreamDestroy(cs);
                if (ce != cudaSuccess) return cuda_fail(e, ce, "cudaGraphInstantiate");
                e->graph_merges = e->d.n_tiles;  // the capture froze the stream pointer, n_tiles and the grids
                e->graph_tiles = e->d.tiles;
            }
            while (batch > 0) {
                CK(cudaGraphLaunch(e->graph, s));
                batch -= G;
            }
        } else {
            for (int i = 0; i < batch; ++i) {
                rc = enqueue_iteration(e, s);
                if (rc != STBPE_OK) return rc;
            }
        }
        if (todo > 0) {  // stop early when a stop rule fired
            CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
            CK(cudaStreamSynchronize(s));
            if (h.stopped) break;
        }
    }
    // one more selection decides the stop reason without applying anything when the target is reached
    select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 1, 0, e->cand);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(s));
    return check_device_error(e, s);
}

// Same loop as stbpe_train, launched kernel by kernel with CUDA events around every launch so
// that a caller can attribute device time to the three kernels (select / merge / refresh).
STBPE_VISIBLE int stbpe_train_timed(stbpe_engine *e, int32_t n_merges, float *kernel_ms, void *stream) {
    if (!e || n_merges < 0 || !kernel_ms) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (!e->counted) return fail(e, STBPE_E_STATE, "count the pairs before training");
    if (e->cfg.world_size > 1) return fail(e, STBPE_E_STATE, "single-rank entry point");
    DevState h;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    i64 target = (i64)h.merges_done + n_merges;
    if (target > e->cfg.max_merges) target = e->cfg.max_merges;
    set_target_kernel<<<1, 1, 0, s>>>(e->d, (int)target);
    CK(cudaGetLastError());
    const int todo = (int)(target - h.merges_done);
    const int P = 128;
    std::vector<cudaEvent_t> ev(4 * P);
    for (auto &x : ev) CK(cudaEventCreate(&x));
    kernel_ms[0] = kernel_ms[1] = kernel_ms[2] = kernel_ms[3] = 0.f;
    int rc = STBPE_OK;
    cudaEvent_t r0, r1;
    CK(cudaEventCreate(&r0));
    CK(cudaEventCreate(&r1));
    for (int base = 0, n = 0; base < todo && rc == STBPE_OK; base += n) {
        {
            int did = 0;
            const bool had_filter = e->filter_valid;
            cudaEventRecord(r0, s);
            rc = maybe_repack(e, false, &did, s);
            cudaEventRecord(r1, s);
            cudaEventSynchronize(r1);
            if (did || had_filter != e->filter_valid) {  // a re-pack and / or a rebuild of the pair filter
                float ms = 0.f;
                cudaEventElapsedTime(&ms, r0, r1);
                kernel_ms[3] += ms;
            }
            if (rc != STBPE_OK) break;
        }
        const int step = (e->filter_valid || e->d.n_tiles < 64) ? P : 32;
        n = todo - base < step ? todo - base : step;
        for (int i = 0; i < n && rc == STBPE_OK; ++i) {
            cudaEventRecord(ev[4 * i], s);
            select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 1, 0, e->cand);
            cudaEventRecord(ev[4 * i + 1], s);
            rc = launch_merge(e, false, s);
            cudaEventRecord(ev[4 * i + 2], s);
            if (rc == STBPE_OK) rc = launch_refresh(e, 0, s);
            cudaEventRecord(ev[4 * i + 3], s);
        }
        cudaStreamSynchronize(s);
        for (int i = 0; i < n && rc == STBPE_OK; ++i)
            for (int k = 0; k < 3; ++k) {
                float ms = 0.f;
                cudaEventElapsedTime(&ms, ev[4 * i + k], ev[4 * i + k + 1]);
                kernel_ms[k] += ms;
            }
    }
    for (auto &x : ev) cudaEventDestroy(x);
    cudaEventDestroy(r0);
    cudaEventDestroy(r1);
    if (rc != STBPE_OK) return rc;
    select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 1, 0, e->cand);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(s));
    return check_device_error(e, s);
}

STBPE_VISIBLE int stbpe_get_state(stbpe_engine *e, stbpe_state *out, void *stream) {
    if (!e || !out) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    DevState h;
    CK(cudaMemcpyAsync(&h, e->d.st, sizeof(h), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    out->merges_done = h.merges_done;
    out->stop_reason = h.stopped ? h.stop_reason : STBPE_RUNNING;
    out->live_tokens = e->recs_stale ? e->n_tokens : h.n_live;
    out->table_keys = (i64)h.n_keys;
    out->table_slots = (i64)e->slots;
    out->device_error = h.error;
    out->n_tiles = e->d.n_tiles;
    out->fixups = h.n_fixups;
    out->repacks = e->repacks;
    out->work_tiles = h.n_work;
    out->count_kernel_ms = e->count_ms;
    out->count_convert_ms = e->convert_ms;
    out->tile_bytes_in = (i64)h.tile_bytes_in;
    out->tile_bytes_out = (i64)h.tile_bytes_out;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_get_merges(stbpe_engine *e, int32_t first, int32_t n, int32_t *merges,
                                   int64_t *counts, int64_t *live_before) {
    if (!e || first < 0 || n < 0 || first + n > e->cfg.max_merges || (n > 0 && !merges))
        return fail(e, STBPE_E_BADARG, "bad merge range");
    CK(cudaSetDevice(e->cfg.device));
    if (n == 0) return STBPE_OK;
    CK(cudaMemcpy(merges, e->d.merges + 2 * first, (size_t)n * 2 * sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (counts) CK(cudaMemcpy(counts, e->d.merge_counts + first, (size_t)n * sizeof(i64), cudaMemcpyDeviceToHost));
    if (live_before) CK(cudaMemcpy(live_before, e->d.live_before + first, (size_t)n * sizeof(i64), cudaMemcpyDeviceToHost));
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_export_histogram(stbpe_engine *e, uint64_t *keys, int64_t *counts, int64_t cap,
                                         int64_t *n_out, void *stream) {
    if (!e || !n_out || cap < 0) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    u64 *tk = nullptr;
    i64 *tc = nullptr;
    CK(cudaMallocAsync((void **)&tk, (size_t)(cap > 0 ? cap : 1) * sizeof(u64), s));
    CK(cudaMallocAsync((void **)&tc, (size_t)(cap > 0 ? cap : 1) * sizeof(i64), s));
    CK(cudaMemsetAsync(&e->d.st->export_n, 0, sizeof(i64), s));
    export_table_kernel<<<e->sm_count * 8, 256, 0, s>>>(e->d, tk, tc, cap);
    CK(cudaGetLastError());
    i64 n = 0;
    CK(cudaMemcpyAsync(&n, &e->d.st->export_n, sizeof(i64), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    *n_out = n;
    int rc = STBPE_OK;
    if (n > cap) {
        rc = fail(e, STBPE_E_CAPACITY, "pair workspace capacity exceeded");
    } else if (n > 0) {
        size_t tmp_bytes = 0;
        cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, tk, (u64 *)keys, tc, (i64 *)counts, (int)n, 0, 64, s);
        void *tmp = nullptr;
        CK(cudaMallocAsync(&tmp, tmp_bytes ? tmp_bytes : 16, s));
        cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, tk, (u64 *)keys, tc, (i64 *)counts, (int)n, 0, 64, s);
        CK(cudaGetLastError());
        CK(cudaFreeAsync(tmp, s));
    }
    CK(cudaFreeAsync(tk, s));
    CK(cudaFreeAsync(tc, s));
    CK(cudaStreamSynchronize(s));
    return rc;
}

STBPE_VISIBLE int stbpe_export_ties(stbpe_engine *e, int64_t count, uint64_t *keys, int64_t cap,
                                    int64_t *n_out, void *stream) {
    if (!e || !n_out || cap < 0 || (cap > 0 && !keys)) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    CK(cudaMemsetAsync(&e->d.st->export_n, 0, sizeof(i64), s));
    export_ties_kernel<<<e->sm_count * 8, 256, 0, s>>>(e->d, count, (u64 *)keys, cap);
    CK(cudaGetLastError());
    i64 n = 0;
    CK(cudaMemcpyAsync(&n, &e->d.st->export_n, sizeof(i64), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    *n_out = n;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_export_stream(stbpe_engine *e, int32_t *ids, int64_t cap, int64_t *n_out,
                                      void *stream) {
    if (!e || !n_out) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    int rc = prepare_stream_state(e, s);
    if (rc != STBPE_OK) return rc;
    const int nt = e->d.n_tiles;
    *n_out = 0;
    if (nt == 0) return STBPE_OK;
    i64 *dl = nullptr;
    CK(cudaMallocAsync((void **)&dl, (size_t)(nt + 1) * sizeof(i64), s));
    tile_lens_kernel<<<(nt + 255) / 256, 256, 0, s>>>(e->d, dl);
    CK(cudaGetLastError());
    std::vector<i64> lens(nt + 1), off(nt + 1);
    CK(cudaMemcpyAsync(lens.data(), dl, (size_t)nt * sizeof(i64), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    off[0] = 0;
    for (int t = 0; t < nt; ++t) off[t + 1] = off[t] + lens[t];
    *n_out = off[nt];
    if (off[nt] > cap) {
        cudaFreeAsync(dl, s);
        return fail(e, STBPE_E_CAPACITY, "export buffer too small");
    }
    CK(cudaMemcpyAsync(dl, off.data(), (size_t)(nt + 1) * sizeof(i64), cudaMemcpyHostToDevice, s));
    export_stream_kernel<<<e->sm_count * 4, 256, 0, s>>>(e->d, dl, ids);
    CK(cudaGetLastError());
    CK(cudaFreeAsync(dl, s));
    CK(cudaStreamSynchronize(s));
    return STBPE_OK;
}

// ------------------------------------------------------------------------------- multi-GPU
STBPE_VISIBLE int stbpe_mg_set_buffers(stbpe_engine *e, void *outbox, void *inbox, int64_t cap_per_peer) {
    if (!e || !outbox || !inbox || cap_per_peer < 1) return fail(e, STBPE_E_BADARG, "bad exchange buffers");
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    e->d.outbox = (Slot *)outbox;
    e->d.inbox = (Slot *)inbox;
    e->d.cap_per_peer = cap_per_peer;
    CK(cudaSetDevice(e->cfg.device));
    outbox_reset_kernel<<<1, 64>>>(e->d);
    CK(cudaGetLastError());
    CK(cudaDeviceSynchronize());
    return STBPE_OK;
}

static int launch_drain(stbpe_engine *e, cudaStream_t s) {
    if (!e->d.outbox || e->d.cap_per_peer < 1) return fail(e, STBPE_E_STATE, "call stbpe_mg_set_buffers first");
    drain_ltable_kernel<<<e->sm_count * 2, 256, 0, s>>>(e->d);
    CK(cudaGetLastError());
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_count_local(stbpe_engine *e, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    int rc = launch_count(e, true, s);
    if (rc != STBPE_OK) return rc;
    rc = launch_drain(e, s);
    if (rc != STBPE_OK) return rc;
    e->counted = true;
    return STBPE_OK;
}

// exchange-only round of the initial histogram: drains what the first round had to keep
STBPE_VISIBLE int stbpe_mg_drain_only(stbpe_engine *e, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    return launch_drain(e, s);
}

STBPE_VISIBLE int stbpe_mg_merge_local(stbpe_engine *e, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    int rc = launch_merge(e, true, s);
    if (rc != STBPE_OK) return rc;
    return launch_drain(e, s);
}

STBPE_VISIBLE int stbpe_mg_apply_inbox(stbpe_engine *e, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    apply_inbox_kernel<<<e->sm_count * 4, 256, 0, s>>>(e->d);
    CK(cudaGetLastError());
    const int all = e->full_refresh_pending ? 1 : 0;
    e->full_refresh_pending = false;
    return launch_refresh(e, all, s);
}

STBPE_VISIBLE int stbpe_mg_candidate(stbpe_engine *e, void *cand_dev, void *stream) {
    if (!e || !cand_dev) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 2, 0, (i64 *)cand_dev);
    CK(cudaGetLastError());
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_commit(stbpe_engine *e, const void *all_cands_dev, void *stream) {
    if (!e || !all_cands_dev) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    commit_kernel<<<1, 1, 0, s>>>(e->d, (const i64 *)all_cands_dev, e->cfg.max_merges);
    CK(cudaGetLastError());
    return STBPE_OK;
}


// ------------------------------------------------------------------ first count of a 16-bit vocabulary, several ranks
// Every rank partitions the pairs of its own rows (first pass); after a barrier that the caller
// provides, the owner of a partition counts it out of every rank's regions over NVLink peer memory
// (second pass).  The next count round (stbpe_mg_count_local, or round 0 of stbpe_mg_peer_run /
// stbpe_mg_run) then finds the table filled and only exchanges, refreshes and selects.
STBPE_VISIBLE int stbpe_mg_wide_export(stbpe_engine *e, void *handle_out64) {
    if (!e || !handle_out64) return STBPE_E_BADARG;
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    if (e->cfg.world_size > STBPE_MAX_PEERS) return fail(e, STBPE_E_BADARG, "at most 16 ranks share buffers");
    if (e->cfg.base_vocab > 65536) return fail(e, STBPE_E_STATE, "the partitioned count needs a vocabulary of at most 65 536 ids");
    CK(cudaSetDevice(e->cfg.device));
    int rc = wide_alloc(e);
    if (rc != STBPE_OK) return rc;
    cudaIpcMemHandle_t h;
    CK(cudaIpcGetMemHandle(&h, e->wide_block));
    memcpy(handle_out64, &h, sizeof(h));
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_wide_open(stbpe_engine *e, const void *handles, int32_t n_handles) {
    if (!e || !handles) return STBPE_E_BADARG;
    if (!e->wide_block) return fail(e, STBPE_E_STATE, "call stbpe_mg_wide_export first");
    if (n_handles != e->cfg.world_size) return fail(e, STBPE_E_BADARG, "one handle per rank is needed");
    if (e->wide_open) return STBPE_OK;
    CK(cudaSetDevice(e->cfg.device));
    e->wide_peers.world = e->cfg.world_size;
    e->wide_peers.rank = e->cfg.rank;
    for (int r = 0; r < n_handles; ++r) {
        if (r == e->cfg.rank) {
            e->wide_peers.block[r] = e->wide_block;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * sizeof(h), sizeof(h));
        void *p = nullptr;
        CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        e->wide_mapped[r] = p;
        e->wide_peers.block[r] = (const unsigned char *)p;
    }
    e->wide_open = true;
    return STBPE_OK;
}

// ranks of one process: the allocations are handed over as plain device pointers
STBPE_VISIBLE int stbpe_mg_wide_block(stbpe_engine *e, void **out) {
    if (!e || !out) return STBPE_E_BADARG;
    if (!e->wide_block) return fail(e, STBPE_E_STATE, "call stbpe_mg_wide_export first");
    *out = e->wide_block;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_wide_set(stbpe_engine *e, const void *const *blocks, int32_t n) {
    if (!e || !blocks) return STBPE_E_BADARG;
    if (!e->wide_block) return fail(e, STBPE_E_STATE, "call stbpe_mg_wide_export first");
    if (n != e->cfg.world_size) return fail(e, STBPE_E_BADARG, "one block per rank is needed");
    e->wide_peers.world = e->cfg.world_size;
    e->wide_peers.rank = e->cfg.rank;
    for (int r = 0; r < n; ++r) {
        if (r != e->cfg.rank && !blocks[r]) return fail(e, STBPE_E_BADARG, "null block");
        e->wide_peers.block[r] = r == e->cfg.rank ? e->wide_block : (const unsigned char *)blocks[r];
    }
    e->wide_open = true;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_wide_pass1(stbpe_engine *e, int32_t *ok, void *stream) {
    if (!e || !ok) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    *ok = 0;
    CK(cudaSetDevice(e->cfg.device));
    if (!e->wide_open) return fail(e, STBPE_E_STATE, "call stbpe_mg_wide_open first");
    const bool fresh = e->recs_stale;
    int rc = count_prologue(e, s);
    if (rc != STBPE_OK) return rc;
    if (e->only_bytes || e->d.n_tiles < 1 || !fresh) {
        // nothing to partition here (no rows on this rank, or bytes): an empty first pass, the peers still read it
        CK(cudaMemsetAsync(e->parts.fill, 0, wide_fill_bytes(e->parts.n_cta), s));
        CK(cudaMemsetAsync(e->wide_dense, 0, 65536 * sizeof(u64), s));
        CK(cudaStreamSynchronize(s));
        *ok = e->d.n_tiles < 1 ? 1 : 0;
        return STBPE_OK;
    }
    int good = 0;
    rc = wide_pass1(e, &good, s);
    *ok = good;
    return rc;
}

STBPE_VISIBLE int stbpe_mg_wide_pass2(stbpe_engine *e, void *stream) {
    if (!e) return STBPE_E_BADARG;
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    if (!e->wide_open) return fail(e, STBPE_E_STATE, "call stbpe_mg_wide_open first");
    const int world = e->cfg.world_size, n_cta = e->parts.n_cta;
    CK(cudaEventRecord(e->ev0, s));
    dense_peers_to_table_kernel<<<256, 256, 0, s>>>(e->d, e->wide_peers, n_cta);
    CK(cudaGetLastError());
    const int owned = (STBPE_PARTS - e->cfg.rank + world - 1) / world;  // partitions rank, rank + world, ...
    for (int i = 0; i < owned; i += e->part_group) {
        const int n = owned - i < e->part_group ? owned - i : e->part_group;
        partition_table_peers_kernel<<<n_cta * 2 * n, 1024, 0, s>>>(e->d, e->wide_peers, e->cfg.rank + i * world, world, n_cta);
    }
    CK(cudaGetLastError());
    CK(cudaEventRecord(e->ev1, s));
    CK(cudaEventSynchronize(e->ev1));
    CK(cudaEventElapsedTime(&e->convert_ms, e->ev0, e->ev1));
    e->count_ms += e->convert_ms;
    e->wide_counted = true;
    e->full_refresh_pending = true;
    e->counted = true;
    return check_device_error(e, s);
}

// Unmap the peers' buffers (call on every rank, then synchronise the ranks, before any destroys its engine).
STBPE_VISIBLE int stbpe_mg_wide_close(stbpe_engine *e) {
    if (!e) return STBPE_E_BADARG;
    CK(cudaSetDevice(e->cfg.device));
    CK(cudaDeviceSynchronize());
    for (int r = 0; r < STBPE_MAX_PEERS; ++r) {
        if (e->wide_mapped[r]) {
            CK(cudaIpcCloseMemHandle(e->wide_mapped[r]));
            e->wide_mapped[r] = nullptr;
        }
        if (r != e->cfg.rank) e->wide_peers.block[r] = nullptr;
    }
    e->wide_open = false;
    return STBPE_OK;
}

// ------------------------------------------------------------------ rounds over peer memory
// The exchange of a round done by the kernels themselves: every rank owns a mailbox that its peers
// map through CUDA IPC; drain_peer_kernel stores the deltas into the owners' mailboxes,
// select_kernel (mode 3) stores the candidate into every mailbox, and apply_peer_kernel /
// the tail of select_kernel wait (bounded, two seconds) for the senders' flags.  A round is six launches
// and nothing else, so batches of rounds replay as one CUDA graph.  One rank per GPU only.
STBPE_VISIBLE int stbpe_mg_peer_export(stbpe_engine *e, int64_t cap_per_peer, void *handle_out64) {
    if (!e || !handle_out64 || cap_per_peer < 1) return STBPE_E_BADARG;
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    if (e->cfg.world_size > STBPE_MAX_PEERS) return fail(e, STBPE_E_BADARG, "at most 16 ranks share mailboxes");
    if (e->d.cap_per_peer != 0 && e->d.cap_per_peer != cap_per_peer)
        return fail(e, STBPE_E_STATE, "exchange buffers of another capacity are already set");
    CK(cudaSetDevice(e->cfg.device));
    if (!e->mail_own) {
        const size_t bytes = STBPE_MAIL_HEADER_BYTES + (size_t)e->cfg.world_size * (cap_per_peer + 1) * sizeof(Slot);
        cudaError_t c = dev_alloc(e, &e->mail_own, bytes);
        if (c != cudaSuccess) return cuda_fail(e, c, "cudaMalloc mailbox");
        CK(cudaMemset(e->mail_own, 0, bytes));
        CK(cudaDeviceSynchronize());
        e->d.cap_per_peer = cap_per_peer;
    }
    cudaIpcMemHandle_t h;
    CK(cudaIpcGetMemHandle(&h, e->mail_own));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle_out64, &h, sizeof(h));
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_peer_open(stbpe_engine *e, const void *handles, int32_t n_handles) {
    if (!e || !handles) return STBPE_E_BADARG;
    if (!e->mail_own) return fail(e, STBPE_E_STATE, "call stbpe_mg_peer_export first");
    if (n_handles != e->cfg.world_size) return fail(e, STBPE_E_BADARG, "one handle per rank is needed");
    if (e->peers_open) return STBPE_OK;
    CK(cudaSetDevice(e->cfg.device));
    for (int r = 0; r < n_handles; ++r) {
        if (r == e->cfg.rank) {
            e->d.mail[r] = e->mail_own;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * sizeof(h), sizeof(h));
        void *p = nullptr;
        CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        e->mail_mapped[r] = p;
        e->d.mail[r] = (unsigned char *)p;
    }
    e->peers_open = true;
    return STBPE_OK;
}

// The same set-up for ranks that live in one process (one GPU each, peer access between the devices
// enabled by the caller): the mailboxes are handed over as plain device pointers.
STBPE_VISIBLE int stbpe_mg_peer_mailbox(stbpe_engine *e, void **out) {
    if (!e || !out) return STBPE_E_BADARG;
    if (!e->mail_own) return fail(e, STBPE_E_STATE, "call stbpe_mg_peer_export first");
    *out = e->mail_own;
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_peer_set(stbpe_engine *e, const void *const *mailboxes, int32_t n) {
    if (!e || !mailboxes) return STBPE_E_BADARG;
    if (!e->mail_own) return fail(e, STBPE_E_STATE, "call stbpe_mg_peer_export first");
    if (n != e->cfg.world_size) return fail(e, STBPE_E_BADARG, "one mailbox per rank is needed");
    for (int r = 0; r < n; ++r) {
        if (r != e->cfg.rank && !mailboxes[r]) return fail(e, STBPE_E_BADARG, "null mailbox");
        e->d.mail[r] = r == e->cfg.rank ? e->mail_own : (unsigned char *)mailboxes[r];
    }
    e->peers_open = true;
    return STBPE_OK;
}

// Unmap the peers' mailboxes (call on every rank, then synchronise the ranks, before any of them
// destroys its engine).
STBPE_VISIBLE int stbpe_mg_peer_close(stbpe_engine *e) {
    if (!e) return STBPE_E_BADARG;
    CK(cudaSetDevice(e->cfg.device));
    CK(cudaDeviceSynchronize());
    if (e->graph) {
        cudaGraphExecDestroy(e->graph);
        e->graph = nullptr;
    }
    for (int r = 0; r < STBPE_MAX_PEERS; ++r) {
        if (e->mail_mapped[r]) {
            CK(cudaIpcCloseMemHandle(e->mail_mapped[r]));
            e->mail_mapped[r] = nullptr;
        }
        if (r != e->cfg.rank) e->d.mail[r] = nullptr;
    }
    e->peers_open = false;
    return STBPE_OK;
}

static int enqueue_peer_round(stbpe_engine *e, bool count_round, cudaStream_t s) {
    int rc = count_round ? launch_count(e, true, s) : launch_merge(e, true, s);
    if (rc != STBPE_OK) return rc;
    drain_peer_kernel<<<e->sm_count * 2, 256, 0, s>>>(e->d);
    CK(cudaGetLastError());
    apply_peer_kernel<<<e->sm_count * 4, 256, 0, s>>>(e->d);
    CK(cudaGetLastError());
    const int all = e->full_refresh_pending ? 1 : 0;
    e->full_refresh_pending = false;
    rc = launch_refresh(e, all, s);
    if (rc != STBPE_OK) return rc;
    select_kernel<<<e->select_grid, STBPE_SELECT_THREADS, 0, s>>>(e->d, 3, 0, e->cand, e->cfg.max_merges);
    CK(cudaGetLastError());
    return STBPE_OK;
}

// first != 0: round 0 counts the local rows.  Enqueues n_rounds rounds; no host synchronisation.
// Every rank must enqueue the same number of rounds.
STBPE_VISIBLE int stbpe_mg_peer_run(stbpe_engine *e, int first, int n_rounds, void *stream) {
    if (!e || n_rounds < 0) return STBPE_E_BADARG;
    if (!e->peers_open) return fail(e, STBPE_E_STATE, "call stbpe_mg_peer_open first");
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    int r = 0;
    if (first && n_rounds > 0) {
        int rc = enqueue_peer_round(e, true, s);
        if (rc != STBPE_OK) return rc;
        e->counted = true;
        ++r;
    }
    const int G = 16;  // rounds per graph replay
    while (r < n_rounds) {
        if (e->use_graph && n_rounds - r >= G) {
            if (e->graph && (e->graph_merges != e->d.n_tiles || e->graph_tiles != e->d.tiles)) {
                cudaGraphExecDestroy(e->graph);
                e->graph = nullptr;
            }
            if (!e->graph) {
                cudaStream_t cs;
                CK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
                cudaGraph_t g;
                CK(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal));
                int rc2 = STBPE_OK;
                e->pdl_now = e->use_pdl;
                for (int i = 0; i < G && rc2 == STBPE_OK; ++i) rc2 = enqueue_peer_round(e, false, cs);
                e->pdl_now = false;
                cudaError_t ce = cudaStreamEndCapture(cs, &g);
                if (rc2 != STBPE_OK) {
                    cudaStreamDestroy(cs);
                    return rc2;
                }
                if (ce != cudaSuccess) {
                    cudaStreamDestroy(cs);
                    return cuda_fail(e, ce, "cudaStreamEndCapture");
                }
                ce = cudaGraphInstantiate(&e->graph, g, 0);
                cudaGraphDestroy(g);
                cudaStreamDestroy(cs);
                if (ce != cudaSuccess) return cuda_fail(e, ce, "cudaGraphInstantiate");
                e->graph_merges = e->d.n_tiles;
                e->graph_tiles = e->d.tiles;
            }
            CK(cudaGraphLaunch(e->graph, s));
            r += G;
        } else {
            int rc = enqueue_peer_round(e, false, s);
            if (rc != STBPE_OK) return rc;
            ++r;
        }
    }
    return STBPE_OK;
}

// ------------------------------------------------------------------ native NCCL round loop
// The rounds of the multi-GPU merge loop issued from C++ on one stream: kernels, an all-to-all of
// the outbox chunks (grouped ncclSend/ncclRecv over NVLink) and an all-gather of the candidates,
// with no Python and no host synchronisation per round.  NCCL is resolved at run time from the
// library that is already loaded in the process (no link-time dependency).
}  // extern "C"

namespace {
struct NcclApi {
    bool ok = false;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclSend) Send = nullptr;
    decltype(&ncclRecv) Recv = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
};
NcclApi &nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
#define NCCL_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name))
            NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
            NCCL_SYM(CommInitRank, "ncclCommInitRank");
            NCCL_SYM(CommDestroy, "ncclCommDestroy");
            NCCL_SYM(GroupStart, "ncclGroupStart");
            NCCL_SYM(GroupEnd, "ncclGroupEnd");
            NCCL_SYM(Send, "ncclSend");
            NCCL_SYM(Recv, "ncclRecv");
            NCCL_SYM(AllGather, "ncclAllGather");
            NCCL_SYM(GetErrorString, "ncclGetErrorString");
#undef NCCL_SYM
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd &&
                     api.Send && api.Recv && api.AllGather && api.GetErrorString;
        }
    }
    return api;
}
void nccl_comm_destroy(void *comm) {
    if (comm && nccl_api().ok) nccl_api().CommDestroy((ncclComm_t)comm);
}
}  // namespace

extern "C" {

#define NCK(call)                                                                              \
    do {                                                                                       \
        ncclResult_t r_ = (call);                                                              \
        if (r_ != ncclSuccess) return fail(e, STBPE_E_CUDA, std::string(#call) + ": " + nccl_api().GetErrorString(r_)); \
    } while (0)

STBPE_VISIBLE int stbpe_mg_nccl_unique_id(void *out128) {
    stbpe_engine *e = nullptr;
    if (!out128) return STBPE_E_BADARG;
    if (!nccl_api().ok) return fail(e, STBPE_E_STATE, "NCCL library not found in this process");
    ncclUniqueId id;
    NCK(nccl_api().GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return STBPE_OK;
}

STBPE_VISIBLE int stbpe_mg_nccl_init(stbpe_engine *e, const void *id128, int64_t cap_per_peer) {
    if (!e || !id128 || cap_per_peer < 1) return STBPE_E_BADARG;
    if (e->cfg.world_size < 2) return fail(e, STBPE_E_STATE, "engine was created with world_size 1");
    if (!nccl_api().ok) return fail(e, STBPE_E_STATE, "NCCL library not found in this process");
    CK(cudaSetDevice(e->cfg.device));
    if (!e->own_boxes) {
        cudaError_t c;
        const size_t n = (size_t)e->cfg.world_size * (cap_per_peer + 1);
        if ((c = dev_alloc(e, &e->d.outbox, n)) != cudaSuccess) return cuda_fail(e, c, "cudaMalloc outbox");
        if ((c = dev_alloc(e, &e->d.inbox, n)) != cudaSuccess) return cuda_fail(e, c, "cudaMalloc inbox");
        CK(cudaMemset(e->d.outbox, 0, n * sizeof(Slot)));
        CK(cudaMemset(e->d.inbox, 0, n * sizeof(Slot)));
        e->d.cap_per_peer = cap_per_peer;
        e->own_boxes = true;
        outbox_reset_kernel<<<1, 64>>>(e->d);
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
    }
    // one communicator per process and device, shared by every engine created later with the same
    // world size and rank (setting one up costs far more than a training run of a small corpus)
    static ncclComm_t g_comm[64] = {};
    static int g_world[64] = {}, g_rank[64] = {};
    const int dev = e->cfg.device;
    if (dev >= 0 && dev < 64 && g_comm[dev] && g_world[dev] == e->cfg.world_size && g_rank[dev] == e->cfg.rank) {
        e->comm = g_comm[dev];
        return STBPE_OK;
    }
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    NCK(nccl_api().CommInitRank(&e->comm, e->cfg.world_size, id, e->cfg.rank));
    if (dev >= 0 && dev < 64) {
        g_comm[dev] = e->comm;
        g_world[dev] = e->cfg.world_size;
        g_rank[dev] = e->cfg.rank;
    }
    return STBPE_OK;
}

// first != 0: round 0 counts the local rows; every other round applies the committed merge (or only
// drains, in an exchange-only round).  n_rounds rounds are enqueued on the stream; no synchronisation.
STBPE_VISIBLE int stbpe_mg_run(stbpe_engine *e, int first, int n_rounds, void *stream) {
    if (!e || n_rounds < 0) return STBPE_E_BADARG;
    if (!e->comm) return fail(e, STBPE_E_STATE, "call stbpe_mg_nccl_init first");
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaSetDevice(e->cfg.device));
    const NcclApi &api = nccl_api();
    const int world = e->cfg.world_size;
    const size_t chunk = (size_t)(e->d.cap_per_peer + 1) * sizeof(Slot);
    for (int r = 0; r < n_rounds; ++r) {
        int rc = (first && r == 0) ? stbpe_mg_count_local(e, stream) : stbpe_mg_merge_local(e, stream);
        if (rc != STBPE_OK) return rc;
        NCK(api.GroupStart());
        for (int p = 0; p < world; ++p) {
            NCK(api.Send((const char *)e->d.outbox + p * chunk, chunk, ncclChar, p, e->comm, s));
            NCK(api.Recv((char *)e->d.inbox + p * chunk, chunk, ncclChar, p, e->comm, s));
        }
        NCK(api.GroupEnd());
        rc = stbpe_mg_apply_inbox(e, stream);
        if (rc != STBPE_OK) return rc;
        rc = stbpe_mg_candidate(e, e->cand, stream);
        if (rc != STBPE_OK) return rc;
        NCK(api.AllGather(e->cand, e->all_cands, 4, ncclInt64, e->comm, s));
        rc = stbpe_mg_commit(e, e->all_cands, stream);
        if (rc != STBPE_OK) return rc;
    }
    return STBPE_OK;
}

}  // extern "C"
