/*
 * Multi-GPU decompositions of the joint attention (one process per GPU).
 *
 *  - head shards and the CFG split are pure index arithmetic: a rank runs the
 *    ordinary attention on its column slice, nothing is exchanged;
 *  - chunked attention: one launch sees a chunk of the keys and merges its
 *    result into a carried state (normalised fp32 output + log2-sum-exp per
 *    row), the building block of split-K and of the ring;
 *  - attention over key runs: the keys of one launch are runs of rows taken
 *    from two buffers, each run optionally guarded by an arrival word that the
 *    kernel waits for (bounded) before it loads the run's rows;
 *  - ring sequence parallelism: every rank keeps its query rows; the K/V rows
 *    of the other ranks are pushed into this GPU's slot pool by their owners'
 *    copy engines while ONE attention launch works through the runs (own
 *    rows, then the slots in ring order) as they arrive. A received chunk
 *    lies in this GPU's own memory before a TMA load reads it. NCCL carries
 *    the set-up exchanges and is the fallback transport.
 *
 * The reference has no multi-GPU code (iris_cuda.cu:122 always uses device
 * 0); these entry points are additions with no counterpart there.
 *
 * NCCL is loaded at run time (dlopen) so that the single-GPU library has no
 * link-time dependency on it.
 */
#include "common.cuh"

#include <cuda.h>
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include "iris_dev.h"
#include "kernels.h"

using namespace iris_b200;

enum { kMaxRanksPlan = 16 };

static unsigned long long host_now_ns(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (unsigned long long)ts.tv_sec * 1000000000ull + (unsigned long long)ts.tv_nsec;
}
static void host_pause(void) { usleep(20); }

/* ------------------------------------------------------------------------
 * Index arithmetic (no device needed)
 * ------------------------------------------------------------------------ */

extern "C" int iris_b200_head_shard(int heads, int nranks, int rank, int *first, int *count) {
    if (heads <= 0 || nranks <= 0 || rank < 0 || rank >= nranks || !first || !count) return IRIS_B200_EINVAL;
    int base = heads / nranks, extra = heads % nranks;     /* the first `extra` ranks take one more */
    *first = rank * base + (rank < extra ? rank : extra);
    *count = base + (rank < extra ? 1 : 0);
    return IRIS_B200_OK;
}

extern "C" int iris_b200_cfg_shard(int batch, int heads, int nranks, int rank,
                                   int *first_entry, int *entry_stride, int *first_head, int *head_count) {
    if (batch <= 0 || heads <= 0 || nranks <= 0 || rank < 0 || rank >= nranks || !first_entry ||
        !entry_stride || !first_head || !head_count)
        return IRIS_B200_EINVAL;
    int groups = batch < nranks ? batch : nranks;          /* GPU groups, one or more entries each */
    int per = nranks / groups;                             /* ranks of a group share its heads */
    if (rank >= groups * per) {                            /* ranks left over by the division idle */
        *first_entry = batch;
        *entry_stride = groups;
        *first_head = 0;
        *head_count = 0;
        return IRIS_B200_OK;
    }
    *first_entry = rank / per;
    *entry_stride = groups;
    return iris_b200_head_shard(heads, per, rank % per, first_head, head_count);
}

extern "C" int iris_b200_seq_shard(int seq, int nranks, int rank, int *first, int *count) {
    return iris_b200_head_shard(seq, nranks, rank, first, count);
}

extern "C" int iris_b200_ring_source(int rank, int step, int nranks) {
    if (nranks <= 0 || rank < 0 || rank >= nranks || step < 0) return -1;
    return ((rank - step) % nranks + nranks) % nranks;
}

extern "C" int iris_b200_ring_plan(int nranks, int max_parts, int *first_step, int *step_count) {
    if (nranks <= 0 || !first_step || !step_count) return -1;
    /* The ring steps of a call are grouped into key parts of the one
     * attention launch: part i covers the steps [first_step[i], first_step[i]
     * + step_count[i]). Parts are what the work list is ordered by, so the
     * chunks that arrive first are worked on first; more than four parts buy
     * nothing (every part costs a partial result per query block). The
     * library's own choice (max_parts <= 0) keeps the last part to the one
     * step that arrives last, because what is left to do after the last
     * arrival is that part's work: the steps before it are spread evenly
     * over the other parts, larger groups first. An explicit max_parts gives
     * that many groups of equal size (+- 1). */
    if (max_parts > 0) {
        const int n = nranks < max_parts ? nranks : max_parts;
        for (int i = 0; i < n; i++) {
            first_step[i] = (int)((long long)nranks * i / n);
            step_count[i] = (int)((long long)nranks * (i + 1) / n) - first_step[i];
        }
        return n;
    }
    const int n = nranks < 4 ? nranks : 4;
    if (n == 1) {
        first_step[0] = 0;
        step_count[0] = nranks;
        return 1;
    }
    const int head = nranks - 1, groups = n - 1;         /* steps and parts before the last */
    int s = 0;
    for (int i = 0; i < groups; i++) {
        const int c = head / groups + (i < head % groups ? 1 : 0);
        first_step[i] = s;
        step_count[i] = c;
        s += c;
    }
    first_step[groups] = s;
    step_count[groups] = 1;
    return n;
}

/* ------------------------------------------------------------------------
 * Chunked attention with carried state
 * ------------------------------------------------------------------------ */

static int attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                           const uint16_t *k, const uint16_t *v, int ldkv,
                           int seq_q, int seq_k, int heads, float scale,
                           const int *key_mask, float *o_state, float *lse_state,
                           int first, int last) {
    if (!require_device("attention_chunk")) return IRIS_B200_ENODEV;
    if (seq_k <= 0 || (last && !out) || (!(first && last) && (!o_state || !lse_state))) {
        set_error(IRIS_B200_EINVAL, "attention_chunk", "bad argument");
        return IRIS_B200_EINVAL;
    }
    int rc = check_attention_args("attention_chunk", out, q, k, v, ldo, ldq, ldkv, seq_q, seq_k, heads, heads, 128);
    if (rc != IRIS_B200_OK) return rc;
    const void *o = out ? (const void *)out : (const void *)q;
    if (!sm100_supported(o, out ? ldo : 8, q, k, v, ldkv, heads, heads, 128, 0, scale) || ldq % 8 != 0 ||
        ((uintptr_t)o_state & 15) != 0) {
        set_error(IRIS_B200_EUNSUPPORTED, "attention_chunk", "arguments outside the tcgen05 kernel's domain");
        return IRIS_B200_EUNSUPPORTED;
    }
    if (seq_q == 0) return IRIS_B200_OK;
    AttnArgs a = attn_args(out, ldo, q, ldq, k, v, ldkv, seq_q, seq_k, heads, scale, key_mask);
    a.acc_mode = first ? (last ? 0 : 1) : (last ? 3 : 2);
    a.o_acc = o_state;
    a.lse_acc = lse_state;
    return launch_attention_sm100(a);
}

extern "C" int iris_b200_attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                                         const uint16_t *k, const uint16_t *v, int ldkv,
                                         int seq_q, int seq_k, int heads, float scale,
                                         const int *key_mask, float *o_state, float *lse_state,
                                         int first, int last) {
    return attention_chunk(out, ldo, q, ldq, k, v, ldkv, seq_q, seq_k, heads, scale, key_mask, o_state, lse_state,
                           first, last);
}

/* ------------------------------------------------------------------------
 * Attention over key runs
 * ------------------------------------------------------------------------ */

/* runs -> launch arguments (views, arrival guards, requested parts). Pure
 * host arithmetic; pointers are only stored. Returns false on a bad run. */
static bool runs_to_args(AttnArgs &a, const iris_b200_key_run *runs, int nruns, int nparts) {
    a.nsrc = nruns;
    a.max_parts = AttnArgs::kMaxParts;
    long long total = 0;
    for (int i = 0; i < nruns; i++) {
        const iris_b200_key_run &r = runs[i];
        if ((r.view != 0 && r.view != 1) || r.rows <= 0 || r.row0 < 0 || r.rows_per_word < 0) return false;
        a.src[i].view = r.view;
        a.src[i].row0 = r.row0;
        a.src[i].rows = r.rows;
        a.src[i].arrive = r.arrive;
        a.src[i].rows_per_word = r.rows_per_word > 0 ? r.rows_per_word : r.rows;
        total += r.rows;
    }
    if (nparts > 1) {
        /* Parts of whole runs, as even in rows as the runs allow: a cut
         * before run i once the rows so far reach the part's share, or when
         * only as many runs are left as parts. */
        if (nparts > nruns) nparts = nruns;
        long long before = 0;
        int part = 1;
        a.part_row[0] = 0;
        for (int i = 1; i < nruns && part < nparts; i++) {
            before += runs[i - 1].rows;
            if (before * nparts >= total * part || nruns - i <= nparts - part) a.part_row[part++] = before;
        }
        a.nparts = part;
    } else if (nparts == 1) {
        a.max_parts = 1;
    }
    return true;
}

extern "C" int iris_b200_attention_runs_plan(const iris_b200_key_run *runs, int nruns, int seq_q, int heads, int nparts,
                                             int sm_count, int *part_tile, int *nkv) {
    if (!runs || nruns <= 0 || nruns > AttnArgs::kMaxSources || nparts < 0 || nparts > AttnArgs::kMaxParts ||
        sm_count <= 0 || !part_tile)
        return -1;
    AttnArgs a = {};
    a.seq_q = seq_q;
    a.heads = heads;
    KeyPlan plan;
    if (!runs_to_args(a, runs, nruns, nparts) || plan_key_parts(a, sm_count, true, &plan) != IRIS_B200_OK) return -1;
    for (int i = 0; i <= plan.nparts; i++) part_tile[i] = plan.part_tile[i];
    if (nkv) *nkv = plan.nkv;
    return plan.nparts;
}

extern "C" int iris_b200_attention_runs(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                                        int seq_q, int heads, float scale,
                                        const uint16_t *k0, const uint16_t *v0, int ld0,
                                        const uint16_t *k1, const uint16_t *v1, int ld1,
                                        const iris_b200_key_run *runs, int nruns,
                                        const uint32_t *arrive_words, uint32_t arrive_value, int nparts) {
    if (!require_device("attention_runs")) return IRIS_B200_ENODEV;
    if (!out || !q || !runs || nruns <= 0 || nruns > AttnArgs::kMaxSources || seq_q < 0 || heads <= 0 ||
        nparts < 0 || nparts > AttnArgs::kMaxParts) {
        set_error(IRIS_B200_EINVAL, "attention_runs", "bad argument");
        return IRIS_B200_EINVAL;
    }
    AttnArgs a = {};
    a.out = out;
    a.ldo = ldo;
    a.q = q;
    a.ldq = ldq;
    a.seq_q = seq_q;
    a.heads = heads;
    a.scale = scale;
    a.k[0] = k0; a.v[0] = v0; a.ldkv[0] = ld0;
    a.k[1] = k1; a.v[1] = v1; a.ldkv[1] = ld1;
    a.arrive = arrive_words;
    a.arrive_seq = arrive_value;
    if (!runs_to_args(a, runs, nruns, nparts)) {
        set_error(IRIS_B200_EINVAL, "attention_runs", "bad key run");
        return IRIS_B200_EINVAL;
    }
    for (int i = 0; i < nruns; i++) {
        const iris_b200_key_run &r = runs[i];
        const uint16_t *kb = r.view == 0 ? k0 : k1, *vb = r.view == 0 ? v0 : v1;
        const int ld = r.view == 0 ? ld0 : ld1;
        if ((r.arrive >= 0 && !arrive_words) ||
            check_attention_args("attention_runs", out, q, kb, vb, ldo, ldq, ld, seq_q, r.rows, heads, heads, 128) !=
                IRIS_B200_OK) {
            set_error(IRIS_B200_EINVAL, "attention_runs", "bad key run");
            return IRIS_B200_EINVAL;
        }
        if (!sm100_supported(out, ldo, q, kb, vb, ld, heads, heads, 128, 0, scale) || ldq % 8 != 0) {
            set_error(IRIS_B200_EUNSUPPORTED, "attention_runs", "arguments outside the tcgen05 kernel's domain");
            return IRIS_B200_EUNSUPPORTED;
        }
    }
    if (seq_q == 0) return IRIS_B200_OK;
    return launch_attention_sm100(a);
}

/* The key runs and the part boundaries (in key rows over the runs) of one
 * rank's attention launch in a ring call: own rows, then the slots in ring
 * order; with equal row counts that fill their slots the slots 1 .. G-1 are
 * one run of adjacent rows guarded by one word per slot. guarded: the slots
 * carry arrival words (copy-engine transport). own_view: 0 = the caller's
 * rows, 1 = slot 0 (rows packed there). Pure host arithmetic. */
static int ring_runs(int me, int G, const int *rows_of, int slot_rows, bool guarded, int own_view, int max_parts,
                     iris_b200_key_run *runs, long long *part_row, int *nparts) {
    const int rows = rows_of[me];
    bool even = true;
    for (int r = 0; r < G; r++) even = even && rows_of[r] == rows;
    int n = 0;
    runs[n++] = iris_b200_key_run{own_view, 0, rows, -1, 0};
    if (G > 1 && even && slot_rows == rows) {
        runs[n++] = iris_b200_key_run{1, slot_rows, (G - 1) * rows, guarded ? 1 : -1, rows};
    } else {
        for (int s = 1; s < G; s++) {
            const int src = iris_b200_ring_source(me, s, G);
            runs[n++] = iris_b200_key_run{1, s * slot_rows, rows_of[src], guarded ? s : -1, 0};
        }
    }
    *nparts = 1;
    if (guarded && G > 1) {
        /* Parts by groups of steps, so that the work list follows the arrivals. */
        long long step_row[kMaxRanksPlan + 1];
        step_row[0] = 0;
        for (int s = 1; s <= G; s++) step_row[s] = step_row[s - 1] + rows_of[iris_b200_ring_source(me, s - 1, G)];
        int first[kMaxRanksPlan], count[kMaxRanksPlan];
        const int np = iris_b200_ring_plan(G, max_parts, first, count);
        for (int i = 0; i < np; i++) part_row[i] = step_row[first[i]];
        *nparts = np;
    }
    return n;
}

extern "C" int iris_b200_ring_launch_plan(int rank, int nranks, const int *rows_of, int heads, int max_parts, int sm_count,
                                          iris_b200_key_run *runs, int *part_tile, int *nkv) {
    if (nranks < 1 || nranks > kMaxRanksPlan || rank < 0 || rank >= nranks || !rows_of || !runs || !part_tile ||
        heads <= 0 || sm_count <= 0)
        return -1;
    int max_rows = 0;
    for (int r = 0; r < nranks; r++) {
        if (rows_of[r] <= 0) return -1;
        max_rows = rows_of[r] > max_rows ? rows_of[r] : max_rows;
    }
    AttnArgs a = {};
    a.seq_q = rows_of[rank];
    a.heads = heads;
    int np = 1;
    const int n = ring_runs(rank, nranks, rows_of, max_rows, true, 0, max_parts, runs, a.part_row, &np);
    long long keep[AttnArgs::kMaxParts + 1];
    for (int i = 0; i < np; i++) keep[i] = a.part_row[i];
    if (!runs_to_args(a, runs, n, 0)) return -1;
    if (np > 1) {
        a.nparts = np;
        for (int i = 0; i < np; i++) a.part_row[i] = keep[i];
    }
    KeyPlan plan;
    if (plan_key_parts(a, sm_count, true, &plan) != IRIS_B200_OK) return -1;
    for (int i = 0; i <= plan.nparts; i++) part_tile[i] = plan.part_tile[i];
    if (nkv) *nkv = plan.nkv;
    return n * 100 + plan.nparts;           /* runs * 100 + parts */
}

extern "C" int iris_b200_set_wait_limit_us(unsigned int us) {
    sm100_set_wait_limit_ns((unsigned long long)us * 1000ull);
    return IRIS_B200_OK;
}

extern "C" int iris_b200_inject_fault(int what) {
    if (what != IRIS_B200_FAULT_STALE_TICKET) return IRIS_B200_EINVAL;
    sm100_inject_stale_ticket();
    return IRIS_B200_OK;
}

/* ------------------------------------------------------------------------
 * Ring sequence parallelism
 *
 * Rank r holds the query rows and the K / V rows of its token block. The
 * chunk of step s (s = 0 .. G-1) is that of rank (r - s) mod G; its owner
 * sends it directly: at step s every rank sends its own rows to rank r + s
 * (NVSwitch gives every pair full bandwidth, so nothing is relayed and no
 * transfer waits for a computation). All transfers are queued on a
 * communication stream, in step order, when the call starts. Transport: the
 * copy engines push the rows from the caller's buffers into the consumer's
 * slot s (pools mapped through CUDA IPC) and then write the call's sequence
 * number into its arrival word s. No SM is spent on communication.
 *
 * The attention of a call is ONE launch whose keys are the runs "own rows,
 * slot 1, ..., slot G-1". The kernel's producer warps wait (bounded) for the
 * arrival word of a slot before its first load, the work list is ordered by
 * groups of steps, and the groups of a query block are merged inside the
 * launch: no per-step launches, no carried state in memory, and a chunk that
 * is late holds up only the CTAs that have nothing else left to do.
 *
 * When the pools cannot be mapped (no peer access), NCCL send / recv moves the
 * chunks instead. NCCL's kernels need SMs, which the persistent attention
 * launch does not give back while it waits, so in that mode all chunks are
 * received first and the attention launch follows on the stream: correct,
 * without overlap.
 * ------------------------------------------------------------------------ */

namespace {

typedef struct { char internal[128]; } NcclId;
typedef void *NcclComm;
typedef int (*FnGetUniqueId)(NcclId *);
typedef int (*FnCommInitRank)(NcclComm *, int, NcclId, int);
typedef int (*FnCommDestroy)(NcclComm);
typedef int (*FnSendRecv)(void *, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*FnGroup)(void);
typedef const char *(*FnErrStr)(int);
typedef int (*FnAllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
typedef int (*FnAsyncError)(NcclComm, int *);
typedef CUresult (*FnStreamValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

enum { kMaxRanks = 16 };

struct Ring {
    void *dl;
    FnGetUniqueId get_id;
    FnCommInitRank init_rank;
    FnCommDestroy destroy;
    FnSendRecv send, recv;
    FnGroup group_start, group_end;
    FnErrStr err_str;
    FnAllGather all_gather;
    FnAsyncError async_error;
    NcclComm comm;
    int rank, nranks;
    int failed;                           /* a call failed half way: the ring is unusable until destroy + init */
    int parts;                            /* key parts of the attention launch, 0: chosen from the rank count */
    cudaStream_t comm_stream;
    cudaEvent_t packed, comm_done;
    /* Slot pool: two sets (used by alternate calls) of nranks slots of
     * slot_rows rows of K | V; slot s of a set receives the chunk of step s
     * (slot 0 holds the packed own rows in the NCCL mode). */
    char *pool;
    size_t slot_bytes;
    int ce;                               /* 0 not decided, 1 copy engines + IPC, -1 NCCL send/recv */
    FnStreamValue32 write32;
    uint32_t *flags;                      /* arrive[kMaxRanks] | seq_words[8] */
    char *peer_pool[kMaxRanks];
    uint32_t *peer_flags[kMaxRanks];
    void *xchg;                           /* device staging of the handle exchange */
    uint32_t seq;
    /* Timeline of the last call (iris_b200_ring_trace) */
    int trace;
    cudaEvent_t t_start, t_push[kMaxRanks], t_kernel[2];
    int t_pushes;
} ring = {};

enum { kFlagArrive = 0, kFlagSeq = kMaxRanks, kFlagWords = kMaxRanks + 8 };

/* staging of the row-parallel out-projection (further down), released with the group */
void proj_close_peers(void);
void proj_release(void);
void gath_close_peers(void);
void gath_release(void);

bool nccl_load(void) {
    if (ring.dl) return true;
    ring.dl = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!ring.dl) ring.dl = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!ring.dl) {
        set_error(IRIS_B200_ECOMM, "dlopen libnccl", dlerror());
        return false;
    }
    ring.get_id = (FnGetUniqueId)dlsym(ring.dl, "ncclGetUniqueId");
    ring.init_rank = (FnCommInitRank)dlsym(ring.dl, "ncclCommInitRank");
    ring.destroy = (FnCommDestroy)dlsym(ring.dl, "ncclCommDestroy");
    ring.send = (FnSendRecv)dlsym(ring.dl, "ncclSend");
    ring.recv = (FnSendRecv)dlsym(ring.dl, "ncclRecv");
    ring.group_start = (FnGroup)dlsym(ring.dl, "ncclGroupStart");
    ring.group_end = (FnGroup)dlsym(ring.dl, "ncclGroupEnd");
    ring.err_str = (FnErrStr)dlsym(ring.dl, "ncclGetErrorString");
    ring.all_gather = (FnAllGather)dlsym(ring.dl, "ncclAllGather");
    ring.async_error = (FnAsyncError)dlsym(ring.dl, "ncclCommGetAsyncError");
    if (!ring.get_id || !ring.init_rank || !ring.destroy || !ring.send || !ring.recv || !ring.group_start ||
        !ring.group_end || !ring.all_gather) {
        set_error(IRIS_B200_ECOMM, "dlsym nccl", "symbol missing");
        return false;
    }
    return true;
}

bool nccl_ok(int rc, const char *what) {
    if (rc == 0) return true;
    set_error(IRIS_B200_ECOMM, what, ring.err_str ? ring.err_str(rc) : "nccl error");
    return false;
}

/* Waits for the library's stream while watching the communicator: an NCCL
 * collective whose peer never joins does not return by itself, but the
 * communicator reports an asynchronous error (or the deadline passes) and
 * the caller gets IRIS_B200_ECOMM instead of a hang on the host. */
bool nccl_wait(cudaStream_t st, double deadline_s, const char *what) {
    cudaEvent_t ev = ring.comm_done;
    if (!cuda_ok(cudaEventRecord(ev, st), "event record")) return false;
    const unsigned long long t0 = host_now_ns();
    for (;;) {
        cudaError_t e = cudaEventQuery(ev);
        if (e == cudaSuccess) return true;
        if (e != cudaErrorNotReady) return cuda_ok(e, what);
        int async = 0;
        if (ring.async_error && ring.async_error(ring.comm, &async) == 0 && async != 0)
            return nccl_ok(async, what);
        if ((double)(host_now_ns() - t0) * 1e-9 > deadline_s) {
            set_error(IRIS_B200_ECOMM, what, "collective did not finish before the deadline");
            return false;
        }
        host_pause();
    }
}

struct IpcPair {
    cudaIpcMemHandle_t pool, flags;
};

/* Unmap the peers' pools; every importer does this before any exporter frees. */
void ce_close_peers(void) {
    for (int r = 0; r < kMaxRanks; r++) {
        if (ring.peer_pool[r]) cudaIpcCloseMemHandle(ring.peer_pool[r]);
        if (ring.peer_flags[r]) cudaIpcCloseMemHandle(ring.peer_flags[r]);
        ring.peer_pool[r] = NULL;
        ring.peer_flags[r] = NULL;
    }
    (void)cudaGetLastError();
}

/* All-gather of one word per rank (the set-up barrier and the vote on the
 * transport). all[r] receives rank r's word. */
bool exchange_word(uint32_t mine, uint32_t *all) {
    char *dev = (char *)ring.xchg;
    uint32_t *send = (uint32_t *)(dev + sizeof(IpcPair) * (kMaxRanks + 1)), *recv = send + 1;
    return cuda_ok(cudaMemcpyAsync(send, &mine, 4, cudaMemcpyHostToDevice, g.stream), "memcpy") &&
           nccl_ok(ring.all_gather(send, recv, 4, 1, ring.comm, g.stream), "ncclAllGather") &&
           nccl_wait(g.stream, 30.0, "ncclAllGather") &&
           cuda_ok(cudaMemcpy(all, recv, 4 * ring.nranks, cudaMemcpyDeviceToHost), "memcpy");
}
bool ring_barrier(void) {
    uint32_t all[kMaxRanks];
    return exchange_word(1u, all);
}

/* Collective: every rank calls it with the same slot size. Allocates (or
 * grows) the slot pool and, for the copy-engine transport, exchanges the IPC
 * handles through an NCCL all-gather and maps the peers' pools and arrival
 * words. The ranks then vote: one rank that could not map a peer puts every
 * rank on the NCCL transport, so nobody waits for a push that never comes.
 * Returns false only when the pool itself cannot be had. */
bool ring_pool(size_t slot_bytes) {
    const int G = ring.nranks;
    if (ring.pool && slot_bytes <= ring.slot_bytes) return true;
    if (!ring.xchg && !cuda_ok(cudaMalloc(&ring.xchg, sizeof(IpcPair) * (kMaxRanks + 1) + 4 * (kMaxRanks + 1)), "malloc"))
        return false;
    bool want = ring.ce >= 0 && G > 1;
    if (want && !ring.write32) {
        void *wr = NULL;
        cudaDriverEntryPointQueryResult q2;
        if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &wr, cudaEnableDefault, &q2) != cudaSuccess ||
            q2 != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            want = false;
        }
        ring.write32 = (FnStreamValue32)wr;
    }
    /* Nobody may still be pushing into a pool that is about to go away. */
    cuda_ok(cudaDeviceSynchronize(), "sync");
    if (G > 1 && !ring_barrier()) return false;          /* every rank's pushes are complete */
    ce_close_peers();
    if (G > 1 && !ring_barrier()) return false;          /* every mapping of the old pools is gone */
    if (ring.pool) cuda_ok(cudaFree(ring.pool), "free");
    ring.pool = NULL;
    ring.slot_bytes = 0;
    if (!ring.flags) {
        if (!cuda_ok(cudaMalloc((void **)&ring.flags, kFlagWords * 4), "malloc") ||
            !cuda_ok(cudaMemset(ring.flags, 0, kFlagWords * 4), "memset"))
            return false;
    }
    if (cudaMalloc((void **)&ring.pool, slot_bytes * G * 2) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error(IRIS_B200_ENOMEM, "ring slot pool", NULL);
        return false;
    }
    ring.slot_bytes = slot_bytes;
    if (G == 1) return true;
    bool mapped = want;
    if (want) {
        IpcPair *dev = (IpcPair *)ring.xchg;
        IpcPair mine, all[kMaxRanks];
        mapped = cudaIpcGetMemHandle(&mine.pool, ring.pool) == cudaSuccess &&
                 cudaIpcGetMemHandle(&mine.flags, ring.flags) == cudaSuccess;
        if (!mapped) memset(&mine, 0, sizeof(mine));
        /* The exchange itself is collective: a rank that failed above still takes part. */
        if (!cuda_ok(cudaMemcpy(dev + kMaxRanks, &mine, sizeof(mine), cudaMemcpyHostToDevice), "memcpy") ||
            !nccl_ok(ring.all_gather(dev + kMaxRanks, dev, sizeof(IpcPair), 1, ring.comm, g.stream), "ncclAllGather") ||
            !nccl_wait(g.stream, 30.0, "ncclAllGather") ||
            !cuda_ok(cudaMemcpy(all, dev, sizeof(IpcPair) * G, cudaMemcpyDeviceToHost), "memcpy"))
            return false;
        for (int r = 0; r < G && mapped; r++) {
            if (r == ring.rank) continue;
            void *pp = NULL, *pf = NULL;
            if (cudaIpcOpenMemHandle(&pp, all[r].pool, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
                cudaIpcOpenMemHandle(&pf, all[r].flags, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
                mapped = false;
            ring.peer_pool[r] = (char *)pp;
            ring.peer_flags[r] = (uint32_t *)pf;
        }
        (void)cudaGetLastError();
    }
    uint32_t votes[kMaxRanks];
    if (!exchange_word(mapped ? 1u : 0u, votes)) return false;
    bool all_mapped = true;
    for (int r = 0; r < G; r++) all_mapped = all_mapped && votes[r] == 1u;
    if (!all_mapped) {
        ce_close_peers();
        if (!ring_barrier()) return false;
    }
    ring.ce = all_mapped ? 1 : -1;
    return true;
}

bool stream_value(FnStreamValue32 fn, cudaStream_t st, const uint32_t *addr, uint32_t value, unsigned flags,
                  const char *what) {
    CUresult r = fn((CUstream)st, (CUdeviceptr)(uintptr_t)addr, value, flags);
    if (r == CUDA_SUCCESS) return true;
    char msg[48];
    snprintf(msg, sizeof(msg), "CUresult %d", (int)r);
    set_error(IRIS_B200_ECUDA, what, msg);
    return false;
}

}  // namespace

extern "C" int iris_b200_ring_unique_id(void *id128) {
    if (!id128) return IRIS_B200_EINVAL;
    if (!nccl_load()) return IRIS_B200_ECOMM;
    NcclId id;
    if (!nccl_ok(ring.get_id(&id), "ncclGetUniqueId")) return IRIS_B200_ECOMM;
    memcpy(id128, &id, sizeof(id));
    return IRIS_B200_OK;
}

extern "C" int iris_b200_ring_init(int rank, int nranks, const void *id128) {
    if (!require_device("ring_init")) return IRIS_B200_ENODEV;
    if (!id128 || nranks < 1 || nranks > kMaxRanks || rank < 0 || rank >= nranks || ring.comm) return IRIS_B200_EINVAL;
    if (!nccl_load()) return IRIS_B200_ECOMM;
    NcclId id;
    memcpy(&id, id128, sizeof(id));
    if (!nccl_ok(ring.init_rank(&ring.comm, nranks, id, rank), "ncclCommInitRank")) {
        ring.comm = NULL;
        return IRIS_B200_ECOMM;
    }
    ring.rank = rank;
    ring.nranks = nranks;
    ring.failed = 0;
    if (ring.ce > 0) ring.ce = 0;
    if (!cuda_ok(cudaStreamCreateWithFlags(&ring.comm_stream, cudaStreamNonBlocking), "stream create"))
        return IRIS_B200_ECUDA;
    cuda_ok(cudaEventCreateWithFlags(&ring.packed, cudaEventDisableTiming), "event create");
    cuda_ok(cudaEventCreateWithFlags(&ring.comm_done, cudaEventDisableTiming), "event create");
    cuda_ok(cudaEventCreate(&ring.t_start), "event create");
    cuda_ok(cudaEventCreate(&ring.t_kernel[0]), "event create");
    cuda_ok(cudaEventCreate(&ring.t_kernel[1]), "event create");
    for (int i = 0; i < kMaxRanks; i++) cuda_ok(cudaEventCreate(&ring.t_push[i]), "event create");
    return g.last_error;
}

extern "C" int iris_b200_ring_configure(int transport, int parts) {
    if (ring.comm || transport < 0 || transport > 1 || parts < 0 || parts > AttnArgs::kMaxParts) return IRIS_B200_EINVAL;
    ring.ce = transport == 1 ? -1 : 0;
    ring.parts = parts;
    return IRIS_B200_OK;
}

extern "C" int iris_b200_ring_transport(void) { return ring.comm ? (ring.ce == 1 ? 0 : 1) : -1; }

extern "C" int iris_b200_ring_trace(int enable) {
    ring.trace = enable ? 1 : 0;
    ring.t_pushes = 0;
    return IRIS_B200_OK;
}

extern "C" int iris_b200_ring_timeline(float *ms, int cap) {
    if (!ring.comm || !ring.trace || !ms || cap < 2) return -1;
    if (!cuda_ok(cudaDeviceSynchronize(), "sync")) return -1;
    int n = 0;
    for (int i = 0; i < 2; i++)
        if (cudaEventElapsedTime(&ms[n], ring.t_start, ring.t_kernel[i]) == cudaSuccess) n++;
    for (int s = 1; s < ring.t_pushes && n < cap; s++)
        if (cudaEventElapsedTime(&ms[n], ring.t_start, ring.t_push[s]) == cudaSuccess) n++;
    (void)cudaGetLastError();
    return n;
}

extern "C" void iris_b200_ring_destroy(void) {
    if (!ring.comm) return;
    cuda_ok(cudaDeviceSynchronize(), "sync");
    ce_close_peers();
    proj_close_peers();
    gath_close_peers();
    /* Every importer has unmapped before any exporter frees. A ring that
     * failed may have lost a peer: no collective is attempted on it. */
    if (ring.nranks > 1 && ring.xchg && !ring.failed) ring_barrier();
    proj_release();
    gath_release();
    if (ring.pool) cuda_ok(cudaFree(ring.pool), "free");
    if (ring.flags) cuda_ok(cudaFree(ring.flags), "free");
    if (ring.xchg) cuda_ok(cudaFree(ring.xchg), "free");
    ring.pool = NULL;
    ring.slot_bytes = 0;
    ring.flags = NULL;
    ring.xchg = NULL;
    if (ring.ce > 0) ring.ce = 0;
    ring.seq = 0;
    ring.destroy(ring.comm);
    ring.comm = NULL;
    cuda_ok(cudaEventDestroy(ring.packed), "event destroy");
    cuda_ok(cudaEventDestroy(ring.comm_done), "event destroy");
    cuda_ok(cudaEventDestroy(ring.t_start), "event destroy");
    cuda_ok(cudaEventDestroy(ring.t_kernel[0]), "event destroy");
    cuda_ok(cudaEventDestroy(ring.t_kernel[1]), "event destroy");
    for (int i = 0; i < kMaxRanks; i++) cuda_ok(cudaEventDestroy(ring.t_push[i]), "event destroy");
    cuda_ok(cudaStreamDestroy(ring.comm_stream), "stream destroy");
}

/* rows_of[r]: token rows of rank r. q, k, v: this rank's rows, row stride
 * ldi. Slot layout: [slot_rows, 2 * heads * 128] (K | V). */
/* Host estimate for the key-part choice of a ring call: the step-s chunk is pushed s-th by its owner (copy engine,
 * ~0.5 GB/ms measured, plus a start-up of ~10 us) and is needed once a work item has gone through the chunks before
 * it, own rows first. A work item is one 256-row query block of one head over all keys; the launch works through
 * ceil(items / SMs) rounds at roughly 1.1 PFLOP/s per GPU. True when every chunk is expected to be there in time. */
static bool ring_chunks_arrive_in_time(const int *rows_of, int G, int me, int heads, int sm_count) {
    double total_rows = 0;
    for (int r = 0; r < G; r++) total_rows += rows_of[r];
    const double flops = 4.0 * rows_of[me] * total_rows * heads * 128.0;
    const double items = (double)((rows_of[me] + 255) / 256) * heads;
    const double rounds = items > sm_count ? items / sm_count : 1.0;
    const double item_us = flops / 1.1e15 * 1e6 / rounds;
    double pushed_us = 10.0, done_rows = rows_of[me];
    for (int s = 1; s < G; s++) {
        const int src = iris_b200_ring_source(me, s, G);
        pushed_us += (double)rows_of[src] * heads * 128.0 * 2 * 2 / 0.5e6;      /* K and V rows, bf16, bytes per us */
        if (pushed_us > item_us * done_rows / total_rows) return false;
        done_rows += rows_of[src];
    }
    return true;
}

extern "C" int iris_b200_ring_attention(uint16_t *out, int ldo,
                                        const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                        int ldi, const int *rows_of, int heads, float scale) {
    if (!require_device("ring_attention")) return IRIS_B200_ENODEV;
    if (!ring.comm || !rows_of || !out || !q || !k || !v || heads <= 0) {
        set_error(IRIS_B200_EINVAL, "ring_attention", "ring not initialised or bad argument");
        return IRIS_B200_EINVAL;
    }
    if (ring.failed) {
        set_error(IRIS_B200_ECOMM, "ring_attention", "an earlier call failed: destroy and re-initialise the ring");
        return IRIS_B200_ECOMM;
    }
    const int G = ring.nranks, me = ring.rank;
    const int rows = rows_of[me];
    const size_t width = (size_t)heads * 128;
    int max_rows = 0;
    bool even = true;
    for (int r = 0; r < G; r++) {
        if (rows_of[r] <= 0) {
            set_error(IRIS_B200_EINVAL, "ring_attention", "every rank needs at least one row");
            return IRIS_B200_EINVAL;
        }
        max_rows = rows_of[r] > max_rows ? rows_of[r] : max_rows;
        even = even && rows_of[r] == rows;
    }
    if (check_attention_args("ring_attention", out, q, k, v, ldo, ldi, ldi, rows, rows, heads, heads, 128) != IRIS_B200_OK)
        return IRIS_B200_EINVAL;
    if (!sm100_supported(out, ldo, q, k, v, ldi, heads, heads, 128, 0, scale)) {
        set_error(IRIS_B200_EUNSUPPORTED, "ring_attention", "arguments outside the tcgen05 kernel's domain");
        return IRIS_B200_EUNSUPPORTED;
    }
    const size_t row_bytes = width * 2, slot_pitch = 2 * row_bytes;      /* a slot row is K | V */
    const size_t slot_bytes = (size_t)max_rows * slot_pitch;
    /* Everything that can fail without having enqueued anything comes first:
     * an error return up to here leaves the ring usable. */
    if (G > 1 && !ring_pool(slot_bytes)) {
        ring.failed = 1;                 /* the ranks may no longer agree on the pools */
        return g.last_error ? g.last_error : IRIS_B200_ECOMM;
    }
    const bool ce = G > 1 && ring.ce == 1;
    const int slot_rows = G > 1 ? (int)(ring.slot_bytes / slot_pitch) : 0;
    const uint32_t seq = ++ring.seq;
    /* Slots come in two sets used by alternate calls. A peer pushes the rows
     * of call n + 1 only after its own call n, whose launch ended only after
     * this rank's push of call n had arrived there, and that push was ordered
     * after this rank's call n - 1: the set of call n + 1 was last read here
     * in call n - 1, so no acknowledgement has to travel back. */
    char *set = G > 1 ? ring.pool + (size_t)(seq & 1u) * G * ring.slot_bytes : NULL;
    const size_t set_off = G > 1 ? (size_t)(set - ring.pool) : 0;
    uint32_t *seq_word = G > 1 ? ring.flags + kFlagSeq + (seq & 7u) : NULL;
    const bool trace = ring.trace == 1;
    bool ok = true;

    /* From here on work is enqueued; a failure marks the ring as failed. */
    if (trace) cudaEventRecord(ring.t_start, g.stream);
    if (G > 1) {
        if (ce) {
            /* Every earlier use of the sequence word is ordered before this
             * point on the library's stream. */
            ok = stream_value(ring.write32, g.stream, seq_word, seq, CU_STREAM_WRITE_VALUE_DEFAULT, "write seq");
        }
        if (ok && !ce) {
            /* NCCL wants the rows contiguous: K | V into slot 0. (The copy
             * engines take strided rows as they are; pushing from a packed
             * copy was measured to be no faster, 48 us per 26 MB either way.) */
            ok = cuda_ok(cudaMemcpy2DAsync(set, slot_pitch, k, (size_t)ldi * 2, row_bytes, rows,
                                           cudaMemcpyDeviceToDevice, g.stream), "pack K") &&
                 cuda_ok(cudaMemcpy2DAsync(set + row_bytes, slot_pitch, v, (size_t)ldi * 2, row_bytes, rows,
                                           cudaMemcpyDeviceToDevice, g.stream), "pack V");
        }
        ok = ok && cuda_ok(cudaEventRecord(ring.packed, g.stream), "event record") &&
             cuda_ok(cudaStreamWaitEvent(ring.comm_stream, ring.packed, 0), "stream wait");
    }
    /* All transfers, in step order on one stream: at step s this rank's rows
     * are wanted by rank me + s, which keeps them in its slot s. (Pushes on
     * two streams were measured to share one copy engine and run one after
     * the other anyway, only no longer in the order the steps need them.) */
    for (int s = 1; s < G && ok; s++) {
        const int to = (me + s) % G, from = iris_b200_ring_source(me, s, G);
        cudaStream_t cs = ring.comm_stream;
        if (ce) {
            char *dst = ring.peer_pool[to] + set_off + (size_t)s * ring.slot_bytes;
            if (v == k + width) {
                /* K and V are neighbouring column blocks of one buffer: one copy of K | V rows. */
                ok = cuda_ok(cudaMemcpy2DAsync(dst, slot_pitch, k, (size_t)ldi * 2, 2 * row_bytes, rows,
                                               cudaMemcpyDefault, cs), "push K|V");
            } else {
                ok = cuda_ok(cudaMemcpy2DAsync(dst, slot_pitch, k, (size_t)ldi * 2, row_bytes, rows, cudaMemcpyDefault,
                                               cs), "push K") &&
                     cuda_ok(cudaMemcpy2DAsync(dst + row_bytes, slot_pitch, v, (size_t)ldi * 2, row_bytes, rows,
                                               cudaMemcpyDefault, cs), "push V");
            }
            ok = ok && cuda_ok(cudaMemcpyAsync(ring.peer_flags[to] + kFlagArrive + s, seq_word, 4, cudaMemcpyDefault, cs),
                               "push flag");
            if (trace) {
                cudaEventRecord(ring.t_push[s], cs);
                ring.t_pushes = s + 1;
            }
        } else {
            ok = nccl_ok(ring.group_start(), "ncclGroupStart");
            bool sent = ok && nccl_ok(ring.send(set, (size_t)rows * slot_pitch, 1, to, ring.comm, cs), "ncclSend") &&
                        nccl_ok(ring.recv(set + (size_t)s * ring.slot_bytes, (size_t)rows_of[from] * slot_pitch, 1, from,
                                          ring.comm, cs), "ncclRecv");
            ok = ok && nccl_ok(ring.group_end(), "ncclGroupEnd") && sent;
        }
    }
    if (G > 1 && ok) ok = cuda_ok(cudaEventRecord(ring.comm_done, ring.comm_stream), "event record");
    if (G > 1 && ok && !ce) ok = cuda_ok(cudaStreamWaitEvent(g.stream, ring.comm_done, 0), "stream wait");

    /* The one attention launch: own rows, then the slots in ring order. With
     * equal row counts the slots 1 .. G-1 are one run of adjacent rows (no
     * half-empty tile at every slot boundary), guarded by one word per slot. */
    AttnArgs a = {};
    int rc = IRIS_B200_OK;
    if (ok) {
        a.out = out;
        a.ldo = ldo;
        a.q = q;
        a.ldq = ldi;
        a.seq_q = rows;
        a.heads = heads;
        a.scale = scale;
        a.max_parts = AttnArgs::kMaxParts;
        a.k[0] = k; a.v[0] = v; a.ldkv[0] = ldi;
        if (G > 1) {
            a.k[1] = (const uint16_t *)set;
            a.v[1] = a.k[1] + width;
            a.ldkv[1] = (int)(2 * width);
            a.arrive = ce ? ring.flags + kFlagArrive : NULL;
            a.arrive_seq = seq;
        }
        iris_b200_key_run runs[kMaxRanks];
        long long part_row[AttnArgs::kMaxParts + 1];
        int np = 1;
        /* The library's choice of key parts (ring.parts == 0): ONE part when every chunk is there before a work
         * item is through its own rows - then nothing waits and no partial result is merged (measured at 4 GPUs, two
         * head groups: 0.743 against 0.773 ms) -, else the grouped plan of iris_b200_ring_plan. */
        int max_parts = ring.parts;
        if (max_parts == 0 && ce && G > 1 && ring_chunks_arrive_in_time(rows_of, G, me, heads, g.sm_count)) max_parts = 1;
        const int n = ring_runs(me, G, rows_of, slot_rows, ce, (ce || G == 1) ? 0 : 1, max_parts, runs, part_row, &np);
        ok = runs_to_args(a, runs, n, 0);
        if (np > 1) {
            a.nparts = np;
            for (int i = 0; i < np; i++) a.part_row[i] = part_row[i];
        }
        if (trace) cudaEventRecord(ring.t_kernel[0], g.stream);
        rc = ok ? launch_attention_sm100(a) : IRIS_B200_EINVAL;
        if (trace) cudaEventRecord(ring.t_kernel[1], g.stream);
    }
    /* The transfers of the local rows must not outlive the call. */
    if (G > 1 && ok && ce) ok = cuda_ok(cudaStreamWaitEvent(g.stream, ring.comm_done, 0), "stream wait");
    if (!ok || rc != IRIS_B200_OK) {
        ring.failed = 1;
        return rc != IRIS_B200_OK ? rc : (g.last_error ? g.last_error : IRIS_B200_ECOMM);
    }
    return IRIS_B200_OK;
}

/* ------------------------------------------------------------------------
 * Row-parallel out-projection with the gated residual (head-parallel ranks)
 *
 * After head-parallel attention rank r holds the columns of the attention
 * output that belong to its heads. The block's out-projection
 * (iris_dev_linear_f32 + iris_dev_residual, iris_transformer_flux.c:3811-3812,
 * 3841-3842) then is a GEMM over a slice of the reduction dimension on every
 * rank whose partial sums have to be added across ranks. Here the GEMM's
 * epilogue sends each fp32 tile row straight to the rank that owns the row
 * (plain stores over NVLink into that rank's staging slab for this sender),
 * the last CTA advances the sender's arrival word on every owner, and the
 * owner's residual kernel waits (bounded) for all senders, sums the slabs and
 * applies x += gate * sum to its rows: a reduce-scatter without a collective
 * library call, and no pass over the partial sums in between. Staging comes
 * in two sets used by alternate calls, for the same reason as the ring's
 * slots. Uses the communicator of iris_b200_ring_init() for the set-up
 * exchange only.
 * ------------------------------------------------------------------------ */

namespace {

struct Proj {
    char *stage;                          /* 2 sets x nranks slabs of slab_bytes */
    size_t slab_bytes;
    uint32_t *words;                      /* arrive[kMaxRanks] | seq words[8] | done counter */
    char *peer_stage[kMaxRanks];
    uint32_t *peer_words[kMaxRanks];
    uint32_t seq;
} proj = {};

enum { kProjDone = kMaxRanks + 8, kProjWords = kMaxRanks + 16 };

void proj_close_peers(void) {
    for (int r = 0; r < kMaxRanks; r++) {
        if (r != ring.rank) {
            if (proj.peer_stage[r]) cudaIpcCloseMemHandle(proj.peer_stage[r]);
            if (proj.peer_words[r]) cudaIpcCloseMemHandle(proj.peer_words[r]);
        }
        proj.peer_stage[r] = NULL;
        proj.peer_words[r] = NULL;
    }
    (void)cudaGetLastError();
}

/* Collective, like ring_pool(): staging of at least slab_bytes per sender and
 * set, mapped on every peer. No fallback: without peer access the call fails. */
bool proj_setup(size_t slab_bytes) {
    const int G = ring.nranks;
    if (proj.stage && slab_bytes <= proj.slab_bytes) return true;
    if (!ring.xchg && !cuda_ok(cudaMalloc(&ring.xchg, sizeof(IpcPair) * (kMaxRanks + 1) + 4 * (kMaxRanks + 1)), "malloc"))
        return false;
    cuda_ok(cudaDeviceSynchronize(), "sync");
    if (G > 1 && !ring_barrier()) return false;
    proj_close_peers();
    if (G > 1 && !ring_barrier()) return false;
    if (proj.stage) cuda_ok(cudaFree(proj.stage), "free");
    proj.stage = NULL;
    proj.slab_bytes = 0;
    if (!proj.words) {
        if (!cuda_ok(cudaMalloc((void **)&proj.words, kProjWords * 4), "malloc") ||
            !cuda_ok(cudaMemset(proj.words, 0, kProjWords * 4), "memset"))
            return false;
    }
    if (cudaMalloc((void **)&proj.stage, slab_bytes * G * 2) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error(IRIS_B200_ENOMEM, "out-projection staging", NULL);
        return false;
    }
    proj.slab_bytes = slab_bytes;
    proj.peer_stage[ring.rank] = proj.stage;
    proj.peer_words[ring.rank] = proj.words;
    if (G == 1) return true;
    IpcPair *dev = (IpcPair *)ring.xchg;
    IpcPair mine, all[kMaxRanks];
    bool mapped = cudaIpcGetMemHandle(&mine.pool, proj.stage) == cudaSuccess &&
                  cudaIpcGetMemHandle(&mine.flags, proj.words) == cudaSuccess;
    if (!mapped) memset(&mine, 0, sizeof(mine));
    if (!cuda_ok(cudaMemcpy(dev + kMaxRanks, &mine, sizeof(mine), cudaMemcpyHostToDevice), "memcpy") ||
        !nccl_ok(ring.all_gather(dev + kMaxRanks, dev, sizeof(IpcPair), 1, ring.comm, g.stream), "ncclAllGather") ||
        !nccl_wait(g.stream, 30.0, "ncclAllGather") ||
        !cuda_ok(cudaMemcpy(all, dev, sizeof(IpcPair) * G, cudaMemcpyDeviceToHost), "memcpy"))
        return false;
    for (int r = 0; r < G && mapped; r++) {
        if (r == ring.rank) continue;
        void *ps = NULL, *pw = NULL;
        if (cudaIpcOpenMemHandle(&ps, all[r].pool, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
            cudaIpcOpenMemHandle(&pw, all[r].flags, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            mapped = false;
        proj.peer_stage[r] = (char *)ps;
        proj.peer_words[r] = (uint32_t *)pw;
    }
    (void)cudaGetLastError();
    uint32_t votes[kMaxRanks];
    if (!exchange_word(mapped ? 1u : 0u, votes)) return false;
    for (int r = 0; r < G; r++) mapped = mapped && votes[r] == 1u;
    if (!mapped) {
        set_error(IRIS_B200_ECOMM, "out-projection staging", "a peer's memory cannot be mapped (no peer access)");
        proj_close_peers();
        return false;
    }
    return true;
}

void proj_release(void) {
    proj_close_peers();
    if (proj.stage) cuda_ok(cudaFree(proj.stage), "free");
    if (proj.words) cuda_ok(cudaFree(proj.words), "free");
    proj.stage = NULL;
    proj.words = NULL;
    proj.slab_bytes = 0;
    proj.seq = 0;
}

/* ---- the all-gather of a tensor-parallel block's normalised hidden state ----
 * Two sets (alternate calls) of [rows, dim] bf16 on every rank, mapped on every
 * peer: a rank's LayerNorm stores its rows into all of them. words: one arrival
 * word per sender, then the completion counter of the LayerNorm launch. */
struct Gath {
    char *buf;
    size_t set_bytes;
    uint32_t *words;
    char *peer_buf[kMaxRanks];
    uint32_t *peer_words[kMaxRanks];
    uint32_t seq;
} gath = {};

enum { kGathDone = kMaxRanks, kGathWords = kMaxRanks + 8 };

void gath_close_peers(void) {
    for (int r = 0; r < kMaxRanks; r++) {
        if (r != ring.rank) {
            if (gath.peer_buf[r]) cudaIpcCloseMemHandle(gath.peer_buf[r]);
            if (gath.peer_words[r]) cudaIpcCloseMemHandle(gath.peer_words[r]);
        }
        gath.peer_buf[r] = NULL;
        gath.peer_words[r] = NULL;
    }
    (void)cudaGetLastError();
}

/* Collective, like proj_setup(). */
bool gath_setup(size_t set_bytes) {
    const int G = ring.nranks;
    if (gath.buf && set_bytes <= gath.set_bytes) return true;
    if (!ring.xchg && !cuda_ok(cudaMalloc(&ring.xchg, sizeof(IpcPair) * (kMaxRanks + 1) + 4 * (kMaxRanks + 1)), "malloc"))
        return false;
    cuda_ok(cudaDeviceSynchronize(), "sync");
    if (G > 1 && !ring_barrier()) return false;
    gath_close_peers();
    if (G > 1 && !ring_barrier()) return false;
    if (gath.buf) cuda_ok(cudaFree(gath.buf), "free");
    gath.buf = NULL;
    gath.set_bytes = 0;
    if (!gath.words) {
        if (!cuda_ok(cudaMalloc((void **)&gath.words, kGathWords * 4), "malloc") ||
            !cuda_ok(cudaMemset(gath.words, 0, kGathWords * 4), "memset"))
            return false;
    }
    if (cudaMalloc((void **)&gath.buf, set_bytes * 2) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error(IRIS_B200_ENOMEM, "all-gather buffer", NULL);
        return false;
    }
    gath.set_bytes = set_bytes;
    gath.peer_buf[ring.rank] = gath.buf;
    gath.peer_words[ring.rank] = gath.words;
    if (G == 1) return true;
    IpcPair *dev = (IpcPair *)ring.xchg;
    IpcPair mine, all[kMaxRanks];
    bool mapped = cudaIpcGetMemHandle(&mine.pool, gath.buf) == cudaSuccess &&
                  cudaIpcGetMemHandle(&mine.flags, gath.words) == cudaSuccess;
    if (!mapped) memset(&mine, 0, sizeof(mine));
    if (!cuda_ok(cudaMemcpy(dev + kMaxRanks, &mine, sizeof(mine), cudaMemcpyHostToDevice), "memcpy") ||
        !nccl_ok(ring.all_gather(dev + kMaxRanks, dev, sizeof(IpcPair), 1, ring.comm, g.stream), "ncclAllGather") ||
        !nccl_wait(g.stream, 30.0, "ncclAllGather") ||
        !cuda_ok(cudaMemcpy(all, dev, sizeof(IpcPair) * G, cudaMemcpyDeviceToHost), "memcpy"))
        return false;
    for (int r = 0; r < G && mapped; r++) {
        if (r == ring.rank) continue;
        void *pb = NULL, *pw = NULL;
        if (cudaIpcOpenMemHandle(&pb, all[r].pool, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
            cudaIpcOpenMemHandle(&pw, all[r].flags, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            mapped = false;
        gath.peer_buf[r] = (char *)pb;
        gath.peer_words[r] = (uint32_t *)pw;
    }
    (void)cudaGetLastError();
    uint32_t votes[kMaxRanks];
    if (!exchange_word(mapped ? 1u : 0u, votes)) return false;
    for (int r = 0; r < G; r++) mapped = mapped && votes[r] == 1u;
    if (!mapped) {
        set_error(IRIS_B200_ECOMM, "all-gather buffer", "a peer's memory cannot be mapped (no peer access)");
        gath_close_peers();
        return false;
    }
    return true;
}

void gath_release(void) {
    gath_close_peers();
    if (gath.buf) cuda_ok(cudaFree(gath.buf), "free");
    if (gath.words) cuda_ok(cudaFree(gath.words), "free");
    gath.buf = NULL;
    gath.words = NULL;
    gath.set_bytes = 0;
    gath.seq = 0;
}

}  // namespace

extern "C" int iris_b200_outproj_residual(float *x_rows, const uint16_t *cat, int ldc, const uint16_t *W, int ldw,
                                          const float *gate, const int *rows_of, int k, int dim) {
    if (!require_device("outproj_residual")) return IRIS_B200_ENODEV;
    if (!ring.comm || !x_rows || !cat || !W || !rows_of || k <= 0 || dim <= 0 || dim % 8 != 0 ||
        ((uintptr_t)x_rows & 15) != 0 || (gate && ((uintptr_t)gate & 15) != 0)) {
        set_error(IRIS_B200_EINVAL, "outproj_residual", "group not initialised (iris_b200_ring_init) or bad argument");
        return IRIS_B200_EINVAL;
    }
    if (ring.failed) {
        set_error(IRIS_B200_ECOMM, "outproj_residual", "an earlier call failed: destroy and re-initialise the group");
        return IRIS_B200_ECOMM;
    }
    const int G = ring.nranks, me = ring.rank;
    int row_first[kMaxRanks + 1], max_rows = 0;
    row_first[0] = 0;
    for (int r = 0; r < G; r++) {
        if (rows_of[r] < 0) {
            set_error(IRIS_B200_EINVAL, "outproj_residual", "negative row count");
            return IRIS_B200_EINVAL;
        }
        row_first[r + 1] = row_first[r] + rows_of[r];
        max_rows = rows_of[r] > max_rows ? rows_of[r] : max_rows;
    }
    const int seq_rows = row_first[G];
    const size_t slab_bytes = (((size_t)max_rows * dim * 4) + 255) & ~(size_t)255;
    if (!proj_setup(slab_bytes)) {
        ring.failed = 1;
        return g.last_error ? g.last_error : IRIS_B200_ECOMM;
    }
    const uint32_t seq = ++proj.seq;
    const size_t set_off = (size_t)(seq & 1u) * G * proj.slab_bytes;
    float *slab[kMaxRanks];
    uint32_t *arrive[kMaxRanks];
    for (int q = 0; q < G; q++) {
        /* this rank's slab on owner q, and this rank's arrival word there */
        slab[q] = (float *)(proj.peer_stage[q] + set_off + (size_t)me * proj.slab_bytes);
        arrive[q] = proj.peer_words[q] + me;
    }
    ScatterArgs sc;
    sc.nranks = G;
    sc.row_first = row_first;
    sc.slab = slab;
    sc.arrive = arrive;
    sc.seq = seq;
    sc.done = proj.words + kProjDone;
    int rc = launch_linear_scatter(cat, ldc, W, ldw, seq_rows, k, dim, sc);
    if (rc == IRIS_B200_OK)
        rc = launch_residual_from_slabs(x_rows, (const float *)(proj.stage + set_off), proj.slab_bytes / 4, G, gate,
                                        rows_of[me], dim, proj.words, seq);
    if (rc != IRIS_B200_OK) ring.failed = 1;
    return rc;
}

extern "C" size_t iris_b200_single_block_tp_scratch_bytes(int seq, int heads_local, int mlp_local) {
    if (seq < 0 || heads_local <= 0 || mlp_local <= 0) return 0;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t hw = (size_t)heads_local * 128;
    return up256((size_t)seq * 3 * hw * 2) + up256((size_t)seq * (hw + mlp_local) * 2);
}

extern "C" int iris_b200_single_block_tp(float *x_rows, void *scratch, const uint16_t *w_in, const uint16_t *w_out,
                                         const float *norm_q, const float *norm_k, const float *mod,
                                         const float *rope_cos, const float *rope_sin, const int *rows_of, int dim,
                                         int heads_local, int mlp_local, const int *key_mask) {
    if (!require_device("single_block_tp")) return IRIS_B200_ENODEV;
    if (!ring.comm || !x_rows || !scratch || !w_in || !w_out || !norm_q || !norm_k || !mod || !rope_cos || !rope_sin ||
        !rows_of || dim <= 0 || dim % 128 != 0 || heads_local <= 0 || mlp_local <= 0 || mlp_local % 8 != 0 ||
        ((uintptr_t)scratch & 255) != 0) {
        set_error(IRIS_B200_EINVAL, "single_block_tp", "group not initialised (iris_b200_ring_init) or bad argument");
        return IRIS_B200_EINVAL;
    }
    if (ring.failed) {
        set_error(IRIS_B200_ECOMM, "single_block_tp", "an earlier call failed: destroy and re-initialise the group");
        return IRIS_B200_ECOMM;
    }
    const int G = ring.nranks, me = ring.rank;
    int row_first[kMaxRanks + 1];
    row_first[0] = 0;
    for (int r = 0; r < G; r++) {
        if (rows_of[r] < 0) {
            set_error(IRIS_B200_EINVAL, "single_block_tp", "negative row count");
            return IRIS_B200_EINVAL;
        }
        row_first[r + 1] = row_first[r] + rows_of[r];
    }
    const int seq = row_first[G];
    if (seq == 0) return IRIS_B200_OK;
    const size_t set_bytes = (((size_t)seq * dim * 2) + 255) & ~(size_t)255;
    if (!gath_setup(set_bytes)) {
        ring.failed = 1;
        return g.last_error ? g.last_error : IRIS_B200_ECOMM;
    }
    const uint32_t call = ++gath.seq;
    const size_t set_off = (size_t)(call & 1u) * gath.set_bytes;
    /* 1. LayerNorm of this rank's rows, stored into every rank's copy of the normalised hidden state */
    GatherOut go = {};
    go.n = G;
    for (int q = 0; q < G; q++) {
        go.dst[q] = (uint16_t *)(gath.peer_buf[q] + set_off) + (size_t)row_first[me] * dim;
        go.word[q] = gath.peer_words[q] + me;
    }
    go.seq = call;
    go.done = gath.words + kGathDone;
    int rc = launch_layer_norm_mod_gather(go, x_rows, mod, mod + dim, rows_of[me], dim, 1e-6f);
    /* 2. this rank's heads and MLP columns of the input projection, row tiles as their owners' rows arrive */
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const int hw = heads_local * 128, ldc = hw + mlp_local;
    uint16_t *qkv = static_cast<uint16_t *>(scratch);
    uint16_t *cat = reinterpret_cast<uint16_t *>(static_cast<unsigned char *>(scratch) + up256((size_t)seq * 3 * hw * 2));
    if (rc == IRIS_B200_OK) {
        RowGuard guard = {gath.words, G, row_first, call};
        rc = launch_linear_glu_guarded(qkv, 3 * hw, cat + hw, ldc, (const uint16_t *)(gath.buf + set_off), dim, w_in, seq, dim,
                                       heads_local, mlp_local, norm_q, norm_k, rope_cos, rope_sin, 1e-6f, guard);
    }
    /* 3. attention over all rows for this rank's heads */
    if (rc == IRIS_B200_OK) {
        iris_b200_clear_error();
        iris_dev_attention(cat, ldc, qkv, qkv + hw, qkv + 2 * hw, 3 * hw, seq, seq, heads_local, heads_local, 128,
                           0.08838834764831845f, 0, key_mask);
        rc = iris_b200_last_error();
    }
    if (rc != IRIS_B200_OK) {
        ring.failed = 1;
        return rc;
    }
    /* 4. this rank's columns of the output projection; partial sums to the rows' owners, gated residual there */
    return iris_b200_outproj_residual(x_rows, cat, ldc, w_out, ldc, mod + 2 * dim, rows_of, ldc, dim);
}

/* A device wait ran out inside a ring call (iris_b200_check_device_status
 * reported IRIS_B200_ETIMEOUT): the peers' pushes and this rank's sets are no
 * longer in step. */
void iris_b200::ring_mark_failed(void) {
    if (ring.comm) ring.failed = 1;
}
