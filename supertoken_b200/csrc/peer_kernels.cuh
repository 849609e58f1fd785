// Multi-GPU rounds over NVLink peer memory: the kernels of a round write their results straight
// into the mailboxes of the other ranks (plain peer stores, a flag per sender carrying the round
// number) and wait, bounded, for the flags of the ranks they need.  No library collective and no
// host step inside a round, so a batch of rounds is one CUDA graph.
//
// Why the waits cannot deadlock and chunks cannot be overwritten while in use: a rank's stream runs
// drain(r) -> apply(r) -> select+commit(r) -> drain(r+1).  Nothing before drain(r) waits for a
// peer's round-r data, so every rank reaches its round-r sends once its round r-1 is over.  A peer
// writes my inbox chunk for round r+1 only after its commit(r), which waited for my candidate of
// round r, which I published after my apply(r) had finished reading the chunk; it writes my
// candidate slot for round r+1 only after its apply(r+1), which waited for my drain(r+1), which
// follows my commit(r), the reader of the slot.
//
// These kernels must only be used with one rank per GPU: kernels that wait for one another are not
// guaranteed to make progress as separate launches on one device.
#pragma once
#include "common.cuh"
#include "tile_kernels.cuh"

#define STBPE_PEER_WAIT_NS 2000000000ull  // a peer wait gives up after two seconds

__device__ __forceinline__ u64 global_timer_ns() {
    u64 t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ u64 ld_acquire_sys(const u64 *p) {
    u64 v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(u64 *p, u64 v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Wait until *flag >= want.  Returns false (and records STBPE_DERR_TIMEOUT) when the time limit runs
// out or when another wait of this engine has already given up.
__device__ __forceinline__ bool peer_wait(const u64 *flag, u64 want, DevState *st) {
    if (ld_acquire_sys(flag) >= want) return true;
    const u64 t0 = global_timer_ns();
    for (;;) {
        if (ld_acquire_sys(flag) >= want) return true;
        if (*(volatile unsigned int *)&st->error & STBPE_DERR_TIMEOUT) return false;
        if (global_timer_ns() - t0 > STBPE_PEER_WAIT_NS) {
            atomicOr(&st->error, STBPE_DERR_TIMEOUT);
            return false;
        }
        __nanosleep(100);
    }
}

// Rank-local deltas -> the owners' mailboxes.  Entries that do not fit the chunk stay in the local
// table for the next round, exactly as in the outbox variant (drain_ltable_kernel).  The last CTA to
// finish writes the chunk headers and raises this rank's flag in every mailbox.
__global__ void drain_peer_kernel(EngineDev e) {
    __shared__ int s_last, s_dead;
    DevState *st = e.st;
    MailHeader *own = mail_header(e, e.rank);
    if (threadIdx.x == 0) s_dead = (*(volatile unsigned int *)&st->error & STBPE_DERR_TIMEOUT) != 0;
    __syncthreads();
    const bool dead = s_dead != 0;  // an earlier wait gave up: send nothing, the host reports it
    const unsigned int n = dead ? 0u : st->n_ltouched;
    unsigned int *kept = e.ltouched + (e.lmask + 1);
    for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const unsigned int idx = e.ltouched[i];
        Slot *s = &e.ltable[idx];
        const Slot v = *s;
        if (v.count != 0) {
            const int owner = owner_of(v.key, e.world);
            const i64 j = (i64)atomicAdd(&own->out_count[owner], 1u);
            if (j >= e.cap_per_peer) {
                kept[atomicAdd(&st->n_lkept, 1u)] = idx;
                st->round_incomplete = 1;
                continue;
            }
            mail_chunk(e, owner, e.rank)[1 + j] = v;  // peer store (local when owner == rank)
        }
        s->key = STBPE_EMPTY;
        s->count = 0;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&st->ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (!dead) {
        const unsigned int nk = *(volatile unsigned int *)&st->n_lkept;
        for (unsigned int i = threadIdx.x; i < nk; i += blockDim.x)
            e.ltouched[i] = ((volatile unsigned int *)kept)[i];
        const u64 round = *(volatile u64 *)&own->round + 1;
        if ((int)threadIdx.x < e.world) {
            const int p = threadIdx.x;
            Slot h;
            h.key = (u64) * (volatile unsigned int *)&own->out_count[p];  // keeps counting past the capacity
            h.count = 0;
            mail_chunk(e, p, e.rank)[0] = h;
            own->out_count[p] = 0;
            __threadfence_system();
            st_release_sys(&mail_header(e, p)->inbox_flag[e.rank], round);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            st->n_ltouched = nk;
            st->n_lkept = 0;
        }
    }
    if (threadIdx.x == 0) st->ticket = 0;
}

// Owners add what this round brought.  Every CTA waits for the flags of all senders first.
__global__ void apply_peer_kernel(EngineDev e) {
    __shared__ int s_ok;
    DevState *st = e.st;
    MailHeader *own = mail_header(e, e.rank);
    const u64 round = *(volatile u64 *)&own->round + 1;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < e.world) {
        if (!peer_wait(&own->inbox_flag[threadIdx.x], round, st)) s_ok = 0;
    }
    __shared__ i64 s_n[STBPE_MAX_PEERS];
    if ((int)threadIdx.x < e.world && s_ok) s_n[threadIdx.x] = (i64)__ldcg(&mail_chunk(e, e.rank, threadIdx.x)[0].key);
    __syncthreads();
    if (!s_ok) return;
    for (int p = 0; p < e.world; ++p) {
        const Slot *chunk = mail_chunk(e, e.rank, p);
        i64 n = s_n[p];
        if (n > e.cap_per_peer) {
            n = e.cap_per_peer;
            if (blockIdx.x == 0 && threadIdx.x == 0) st->round_incomplete = 1;
        }
        for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
            const ulonglong2 raw = __ldcg(reinterpret_cast<const ulonglong2 *>(chunk + 1 + i));
            table_add(e, raw.x, (i64)raw.y);
        }
    }
}

// This rank's candidate {key, count, incomplete, 0} into every mailbox (called by the one thread
// that finishes select_kernel, which then commits with commit_from_mailbox: publishing comes before
// any wait on every rank, so the waits cannot block one another).
__device__ __forceinline__ void publish_candidate(const EngineDev &e, u64 key, i64 count, i64 incomplete) {
    const u64 round = *(volatile u64 *)&mail_header(e, e.rank)->round + 1;
    for (int p = 0; p < e.world; ++p) {
        MailHeader *h = mail_header(e, p);
        i64 *c = h->cands[e.rank];
        c[0] = (i64)key;
        c[1] = count;
        c[2] = incomplete;
        c[3] = 0;
    }
    __threadfence_system();
    for (int p = 0; p < e.world; ++p) st_release_sys(&mail_header(e, p)->cand_flag[e.rank], round);
}

// Every rank waits for all candidates of the round and takes the same decision (commit_kernel's
// rule); the round counter advances whatever the decision.  Called by one thread.
__device__ __forceinline__ void commit_from_mailbox(const EngineDev &e, int target) {
    DevState *st = e.st;
    MailHeader *own = mail_header(e, e.rank);
    const u64 round = *(volatile u64 *)&own->round + 1;
    bool ok = true;
    for (int p = 0; p < e.world; ++p) ok &= peer_wait(&own->cand_flag[p], round, st);
    own->round = round;
    st->target = target;
    st->round_incomplete = 0;
    if (!ok) {  // a peer never answered: idle every later kernel of this engine; the host reads the error bit
        st->stopped = 1;
        return;
    }
    if (st->stopped) return;
    u64 bk = STBPE_EMPTY;
    i64 bc = 0;
    bool incomplete = false;
    i64 c[STBPE_MAX_PEERS][3];
#pragma unroll 1
    for (int r = 0; r < e.world; ++r) {  // all loads first, then the comparison chain
        c[r][0] = __ldcg(&own->cands[r][0]);
        c[r][1] = __ldcg(&own->cands[r][1]);
        c[r][2] = __ldcg(&own->cands[r][2]);
    }
    for (int r = 0; r < e.world; ++r) {
        const u64 k = (u64)c[r][0];
        const i64 n = c[r][1];
        incomplete |= c[r][2] != 0;
        if (n > 0 && better(k, n, bk, bc)) {
            bk = k;
            bc = n;
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
