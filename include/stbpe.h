/*
 * stbpe -- B200 (sm_100a) BPE merge-loop engine, C ABI.
 *
 * One engine handle per GPU / rank.  All entry points return an int status
 * (STBPE_OK = 0); stbpe_last_error() gives a message for the last failure on a
 * handle.  No entry point takes or returns a torch type: pointers and sizes only.
 * Pointers marked "host or device" are classified with cudaPointerGetAttributes.
 * Calls on one handle come from one host thread at a time (the reference drives
 * its trainer from a single thread, gpu_tokenizer/bpe_trainer.py:2501).
 *
 * The citations name the reference interface each entry point stands in for
 * (paths relative to the reference project).
 */
#ifndef STBPE_H
#define STBPE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STBPE_OK 0
#define STBPE_E_BADARG 1     /* ValueError / TypeError in the reference (cuda_kernels.py:761-775) */
#define STBPE_E_CAPACITY 2   /* RuntimeError("pair workspace capacity exceeded") (utils.py:619-620) */
#define STBPE_E_TIMEOUT 3    /* a bounded device-side wait gave up */
#define STBPE_E_CUDA 4       /* any CUDA runtime failure; OOM text contains "CUDA out of memory" */
#define STBPE_E_ID_OVERFLOW 5 /* OverflowError: id above the supported range (utils.py:436-439) */
#define STBPE_E_STATE 6      /* call made in the wrong state (e.g. training before counting) */

/* stop reasons reported by stbpe_get_state */
#define STBPE_RUNNING 0
#define STBPE_STOP_TARGET 1     /* requested number of merges reached */
#define STBPE_STOP_NO_PAIRS 2   /* no adjacent pair left (bpe_trainer.py:4304-4308) */
#define STBPE_STOP_LOW_COUNT 3  /* best count < 2 (bpe_trainer.py:2491-2494, :4361-4364) */
#define STBPE_STOP_ERROR 4      /* device error flag set; see stbpe_last_error */

typedef struct stbpe_engine stbpe_engine;

typedef struct stbpe_config {
    int32_t device;          /* CUDA device ordinal */
    int32_t base_vocab;      /* first merge gets id base_vocab (bpe_trainer.py:4365) */
    int64_t max_tokens;      /* capacity of the token stream on this engine */
    int64_t table_slots;     /* pair table capacity, rounded up to a power of two; 0 = auto */
    int32_t max_merges;      /* capacity of the merge log */
    int32_t world_size;      /* >1: pair keys are owned by hash(key) % world_size */
    int32_t rank;
    int32_t reserved;
} stbpe_config;

typedef struct stbpe_state {
    int32_t merges_done;
    int32_t stop_reason;      /* STBPE_RUNNING ... */
    int64_t live_tokens;      /* tokens currently in the stream */
    int64_t table_keys;       /* distinct keys ever inserted into the pair table */
    int64_t table_slots;
    uint32_t device_error;    /* raw device error bits (0 = none) */
    int32_t n_tiles;
    int64_t fixups;           /* dropped partners handled outside the visited tiles (statistics) */
    int64_t repacks;          /* dense re-packs of the stream so far */
    int64_t work_tiles;       /* tiles visited by the last merge (after the pair filter) */
    double count_kernel_ms;   /* device time of the histogram kernel(s) of the last count; on the
                                 16-bit-vocabulary path both passes, i.e. until the pair table is complete */
    double count_convert_ms;  /* 16-bit-vocabulary path only: the part of count_kernel_ms spent in the
                                 second pass (per-partition counting and table inserts; 0 otherwise) */
    int64_t tile_bytes_in;    /* merge kernel, since the last load: bytes of tiles and tile records read ... */
    int64_t tile_bytes_out;   /* ... and bytes of rewritten tile parts and records stored (statistics) */
} stbpe_state;

/* Lifetime.  Replaces GPUBPETrainer's per-fit device contexts and workspaces
 * (gpu_tokenizer/bpe_trainer.py:2907-2934, :224-282). */
int stbpe_create(stbpe_engine **out, const stbpe_config *cfg);
int stbpe_destroy(stbpe_engine *e);
const char *stbpe_last_error(const stbpe_engine *e);
const char *stbpe_version(void);

/* Ingest: pack rows into the flat int32 token stream (bit 31 = first token of a row).
 * Replaces BytePacker.encode_view + the batcher fill + GPUBatchRecord.from_cpu
 * (gpu_tokenizer/cpu_packer.py:17-61, datasets.py:75-84, bpe_trainer.py:137-222).
 * Rows are appended after the rows of earlier calls; empty rows own no pair and
 * vanish.  row_offsets has n_rows+1 entries (host memory), offsets into data.
 * Appending is possible until the first merge has been applied: afterwards the tiles of the
 * stream are no longer dense and the call returns STBPE_E_STATE (call stbpe_reset first).
 * stbpe_reset drops the stream, the table and the merge log. */
int stbpe_reset(stbpe_engine *e);
int stbpe_append_bytes(stbpe_engine *e, const uint8_t *data /* host or device */, int64_t n,
                       const int64_t *row_offsets, int64_t n_rows, void *stream);
int stbpe_append_ids(stbpe_engine *e, const int32_t *ids /* host or device */, int64_t n,
                     const int64_t *row_offsets, int64_t n_rows, void *stream);

/* Full adjacent-pair histogram of the current stream into the pair table.
 * Replaces utils.count_pairs + aggregate_pair_keys (gpu_tokenizer/utils.py:558-635,
 * :709-751).  Clears the table first, so it may also be called after merges to
 * recount from the rewritten stream. */
int stbpe_count_initial(stbpe_engine *e, void *stream);

/* Best pair: maximum count, ties to the smallest packed key (a<<32)|b.
 * Replaces select_best_pair (gpu_tokenizer/trainers/bpe_gpu.py:96-130).  count 0 =
 * empty histogram.  n_ties = number of keys holding the maximum count. */
int stbpe_select_best(stbpe_engine *e, uint64_t *key, int64_t *count, int64_t *n_ties, void *stream);

/* Apply one merge to every row and update the pair table by the +-deltas only.
 * Replaces utils.apply_merge_once + compact_tokens_inplace
 * (gpu_tokenizer/utils.py:413-555, :347-410) followed by the recount of the next
 * loop iteration.  The merge is appended to the merge log with the count the
 * table held for (a, b).  n_matches may be NULL. */
int stbpe_apply_merge(stbpe_engine *e, int32_t a, int32_t b, int32_t new_id, int64_t *n_matches,
                      void *stream);

/* The merge loop (gpu_tokenizer/bpe_trainer.py:4193-4517) run on the device without
 * a host round trip per merge: select -> stop rules -> apply, n_merges times or until a
 * stop rule fires.  Synchronises the stream before returning. */
int stbpe_train(stbpe_engine *e, int32_t n_merges, void *stream);

/* stbpe_train with CUDA events around every kernel launch (no graph replay): kernel_ms[0..3]
 * receive the summed device time of the select, merge and refresh kernels and of the re-packs.  Measurement aid
 * for the per-stage timings the reference records (gpu_tokenizer/bpe_trainer.py:4249-4260,
 * :4385-4396). */
int stbpe_train_timed(stbpe_engine *e, int32_t n_merges, float *kernel_ms, void *stream);

/* Dense re-pack of the token stream (tiles only shrink; stbpe_train does this by itself whenever
 * at most half of the tile capacity in use is live).  force != 0 re-packs regardless.  *did (may
 * be NULL) reports whether it happened.  Replaces nothing in the reference, whose rows are
 * re-compacted by every merge (gpu_tokenizer/utils.py:347-410). */
int stbpe_repack(stbpe_engine *e, int force, int *did, void *stream);

int stbpe_get_state(stbpe_engine *e, stbpe_state *out, void *stream);
/* merges: 2*n int32 (a, b); counts: n int64 (may be NULL); live_before: n int64, live
 * tokens before each merge (may be NULL).  Host pointers. */
int stbpe_get_merges(stbpe_engine *e, int32_t first, int32_t n, int32_t *merges, int64_t *counts,
                     int64_t *live_before);

/* Export of the pair table as the reference returns histograms: unique keys ascending,
 * int64 counts, zero-count keys dropped (gpu_tokenizer/utils.py:709-751).  keys/counts
 * are device pointers with room for cap entries. */
int stbpe_export_histogram(stbpe_engine *e, uint64_t *keys, int64_t *counts, int64_t cap,
                           int64_t *n_out, void *stream);
/* All keys whose count equals `count`, unordered, into keys (device, cap entries); *n_out is
 * their number even when it exceeds cap.  Feeds the seeded random tie-break, which indexes the
 * tied candidates in ascending key order (gpu_tokenizer/bpe_trainer.py:915-923,
 * trainers/bpe_gpu.py:112-123). */
int stbpe_export_ties(stbpe_engine *e, int64_t count, uint64_t *keys, int64_t cap, int64_t *n_out,
                      void *stream);
/* Export of the rewritten stream: ids (device, cap tokens, bit 31 = row start). */
int stbpe_export_stream(stbpe_engine *e, int32_t *ids, int64_t cap, int64_t *n_out, void *stream);

/* Multi-GPU exchange steps (one engine per rank, created with world_size > 1; the collectives
 * are issued by the host between these calls on the same stream).  Together they replace
 * reduce_pair_histograms (gpu_tokenizer/utils.py:863-978): instead of gathering whole histograms,
 * ranks exchange only the +-deltas of a merge, routed to the rank that owns the key
 * (hash(key) % world_size).
 *   stbpe_mg_set_buffers : caller-owned device buffers, each world_size chunks of
 *                          (1 + cap_per_peer) 16-byte entries {key, delta}; entry 0 of a chunk
 *                          holds the entry count.  outbox chunk p goes to rank p (all-to-all with
 *                          equal splits), inbox chunk p comes from rank p.
 *   stbpe_mg_count_local : local histogram of this rank's rows into the outbox (first round)
 *   stbpe_mg_merge_local : apply the current merge to this rank's rows, deltas into the outbox;
 *                          in an exchange-only round it just drains what earlier rounds kept
 *   stbpe_mg_drain_only  : exchange-only round for the initial histogram
 *   stbpe_mg_apply_inbox : add the received deltas into this rank's slice of the pair table
 *   stbpe_mg_candidate   : this rank's best {key, count, incomplete, 0} (4 x int64, device)
 *   stbpe_mg_commit      : takes the all-gathered candidates (world_size x 4 int64); every rank
 *                          reaches the same decision: commit the best pair, stop, or - while any
 *                          rank still holds deltas that did not fit a chunk - run another
 *                          exchange-only round.  No host synchronisation is needed per merge. */
int stbpe_mg_set_buffers(stbpe_engine *e, void *outbox, void *inbox, int64_t cap_per_peer);
int stbpe_mg_count_local(stbpe_engine *e, void *stream);
int stbpe_mg_drain_only(stbpe_engine *e, void *stream);
int stbpe_mg_merge_local(stbpe_engine *e, void *stream);
int stbpe_mg_apply_inbox(stbpe_engine *e, void *stream);
int stbpe_mg_candidate(stbpe_engine *e, void *cand_dev /* 4 x int64 */, void *stream);
int stbpe_mg_commit(stbpe_engine *e, const void *all_cands_dev /* world x 4 int64 */, void *stream);

/* The same rounds issued natively on one stream, without a host call per step: the library
 * resolves NCCL from the process at run time and keeps its own communicator.
 *   stbpe_mg_nccl_unique_id : rank 0 obtains the 128-byte NCCL id, the caller broadcasts it
 *   stbpe_mg_nccl_init      : every rank joins the communicator (and gets exchange buffers of
 *                             cap_per_peer entries per peer if none were set).  The communicator is
 *                             created once per process and device and reused by later engines of the
 *                             same world size and rank (id128 is then ignored)
 *   stbpe_mg_run            : enqueue n_rounds rounds (first != 0: round 0 is the local count); each
 *                             round = local kernel, all-to-all of the chunks (grouped ncclSend/ncclRecv),
 *                             owner insert, candidate, all-gather, commit.  Does not synchronise.
 * Stand in for the NCCL process-group set-up of the reference (gpu_tokenizer/dist/launcher.py:143-182). */
int stbpe_mg_nccl_unique_id(void *out128);
int stbpe_mg_nccl_init(stbpe_engine *e, const void *id128, int64_t cap_per_peer);
int stbpe_mg_run(stbpe_engine *e, int first, int n_rounds, void *stream);

/* The same rounds with the exchange done by the kernels themselves over NVLink peer memory, one
 * process per GPU, no library collective inside a round.  Replaces the histogram reduce of the
 * reference (gpu_tokenizer/utils.py:863-978, one NCCL all-reduce per count) on this path.
 *   stbpe_mg_peer_export : allocates this rank's mailbox (header + one chunk of cap_per_peer entries
 *                          per sender) and returns its 64-byte CUDA IPC handle; the caller gathers the
 *                          handles of all ranks (any host transport)
 *   stbpe_mg_peer_open   : maps the mailboxes of the other ranks (handles: world x 64 bytes, indexed by
 *                          rank; the own entry is ignored)
 *   stbpe_mg_peer_run    : enqueue n_rounds rounds (first != 0: round 0 is the local count); batches of
 *                          16 rounds replay as one CUDA graph.  Every rank must enqueue the same number
 *                          of rounds, and the ranks should start them within a second of one another:
 *                          a kernel waits at most two seconds for a peer's flag, then records a time-out
 *                          that the next stbpe_get_state / error check reports (STBPE_E_TIMEOUT); the
 *                          engine is then unusable.  Does not synchronise.
 *   stbpe_mg_peer_close  : unmaps the peers' mailboxes; call on every rank and synchronise the ranks
 *                          before any of them destroys its engine.
 * At most 16 ranks.  Never run two ranks of one job on the same GPU with these entry points (the
 * kernels of different ranks wait for one another); stbpe_mg_set_buffers + the step-wise entry
 * points above serve that case. */
int stbpe_mg_peer_export(stbpe_engine *e, int64_t cap_per_peer, void *handle_out64);
int stbpe_mg_peer_open(stbpe_engine *e, const void *handles, int32_t n_handles);
int stbpe_mg_peer_run(stbpe_engine *e, int first, int n_rounds, void *stream);
int stbpe_mg_peer_close(stbpe_engine *e);
/* Ranks of one process (one GPU each, peer access enabled by the caller) skip CUDA IPC:
 *   stbpe_mg_peer_mailbox : this rank's mailbox as a device pointer (after stbpe_mg_peer_export)
 *   stbpe_mg_peer_set     : the mailboxes of all ranks as device pointers, indexed by rank. */
int stbpe_mg_peer_mailbox(stbpe_engine *e, void **out);
int stbpe_mg_peer_set(stbpe_engine *e, const void *const *mailboxes, int32_t n);

/* First count of an id stream over a vocabulary of at most 65 536 ids on several ranks of one NVLink
 * domain.  Replaces, for this case, the count + cross-rank reduce of the reference's first loop
 * iteration (gpu_tokenizer/utils.py:558-635 followed by :863-978, which gathers every rank's whole
 * key list): every rank partitions the pairs of its own rows, and the rank that owns a partition
 * (partition modulo world_size, the same rule that owns the keys during the merge loop) counts it out
 * of all ranks' buffers with peer loads.
 *   stbpe_mg_wide_export : allocates this rank's partition buffers and returns their 64-byte CUDA IPC
 *                          handle; the caller gathers the handles of all ranks
 *   stbpe_mg_wide_open   : maps the buffers of the other ranks (world x 64 bytes, indexed by rank)
 *   stbpe_mg_wide_block / stbpe_mg_wide_set : the same for ranks of one process, as device pointers
 *   stbpe_mg_wide_pass1  : partitions this rank's rows; *ok = 0 if the stream does not qualify (bytes,
 *                          an id of 65 536 or more, a full buffer).  Synchronises the stream.
 *   -- the caller synchronises the ranks here (any barrier) and checks that every rank reported ok;
 *      if one did not, all skip the second pass and the ordinary count round does the counting --
 *   stbpe_mg_wide_pass2  : counts the partitions this rank owns.  The next count round
 *                          (stbpe_mg_count_local, or round 0 of stbpe_mg_run / stbpe_mg_peer_run) then
 *                          finds the table filled and only exchanges, refreshes and selects.
 *   stbpe_mg_wide_close  : unmaps the peers' buffers; call on every rank and synchronise the ranks
 *                          before any of them destroys its engine. */
int stbpe_mg_wide_export(stbpe_engine *e, void *handle_out64);
int stbpe_mg_wide_open(stbpe_engine *e, const void *handles, int32_t n_handles);
int stbpe_mg_wide_block(stbpe_engine *e, void **out);
int stbpe_mg_wide_set(stbpe_engine *e, const void *const *blocks, int32_t n);
int stbpe_mg_wide_pass1(stbpe_engine *e, int32_t *ok, void *stream);
int stbpe_mg_wide_pass2(stbpe_engine *e, void *stream);
int stbpe_mg_wide_close(stbpe_engine *e);

/* Stateless operators on padded [B, L] batches resident on the device, with the
 * reference's operator signatures.
 * stbpe_rows_count_pairs  <- utils.count_pairs (gpu_tokenizer/utils.py:691-706): unique
 *   (a, b) rows ascending into pair_keys[cap][2] (rest -1), int64 counts (rest 0), length.
 * stbpe_rows_apply_merge  <- utils.apply_merge_once / cuda_kernels.apply_merge_and_compact
 *   (gpu_tokenizer/utils.py:413-555, cuda_kernels.py:725-832): in place on tokens/valid,
 *   lengths int32[B], spans uint8 [B][L-1] in pre-compaction coordinates (may be NULL). */
int stbpe_rows_count_pairs(const int32_t *tokens, const uint8_t *valid, int64_t B, int64_t L,
                           int32_t *pair_keys, int64_t *pair_counts, int64_t cap,
                           int64_t *length_dev, void *stream);
int stbpe_rows_apply_merge(int32_t *tokens, uint8_t *valid, int32_t *lengths, int64_t B, int64_t L,
                           int32_t a, int32_t b, int32_t new_id, uint8_t *spans, void *stream);

/* stbpe_rows_count_pairs for callers that must not allocate device memory.  It has no
 * counterpart in the reference.  Same inputs, outputs and result as stbpe_rows_count_pairs, but
 * every temporary lives in one fixed block of device memory that is part of the library image
 * (about 5.3 MB, held by every GPU that loads the library until the process exits); the call
 * makes no cudaMalloc / cudaFree / cudaMallocAsync and calls no allocating library routine.
 * Who needs it: a trainer that has already given all device memory to its preallocated
 * workspaces (the reference fills the device up to its --target-util share before the merge
 * loop, so a later allocation is the one that fails), and callers that keep several streams
 * busy and cannot take the device-wide synchronisation a cudaMalloc / cudaFree implies.
 * Limits and rules:
 *   - B*(L-1) must not exceed 65 536 pair positions; larger batches get STBPE_E_CAPACITY and a
 *     message in err (err may be NULL).  Nothing is computed in that case.
 *   - The first call on each device looks up the block's device address
 *     (cudaGetSymbolAddress).  Every call reads the number of unique pairs back to the host and
 *     synchronises the stream, so make no call while the stream is being captured.
 *   - All calls share the block, which keeps the previous call's contents; it is cleared at the
 *     start of each call.  Calls that overlap on the GPU race: serialise them. */
int stbpe_rows_count_pairs_noalloc(const int32_t *tokens, const uint8_t *valid, int64_t B, int64_t L,
                                   int32_t *pair_keys, int64_t *pair_counts, int64_t cap,
                                   int64_t *length_dev, void *stream, char *err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* STBPE_H */
