/*
 * Multi-GPU decompositions of the joint attention (one process per GPU).
 *
 *  - head shards and the CFG split are pure index arithmetic: a rank runs the
 *    ordinary attention on its column slice, nothing is exchanged;
 *  - chunked attention: one launch sees a chunk of the keys and merges its
 *    result into a carried state (normalised fp32 output + log2-sum-exp per
 *    row), the building block of split-K and of the ring;
 *  - ring sequence parallelism: every rank keeps its query rows and walks the
 *    K/V chunks of the other ranks in ring order; the chunks arrive through
 *    NCCL send/recv on a second stream while the attention of earlier chunks
 *    runs. A received chunk lands in this GPU's own memory and is read from
 *    there by ordinary TMA loads.
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

#include "kernels.h"

using namespace iris_b200;

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

extern "C" int iris_b200_ring_plan(int nranks, int even_rows, int *first_step, int *step_count) {
    if (nranks <= 0 || !first_step || !step_count) return -1;
    /* With many ranks a step is a small problem whose fixed costs (pipeline
     * fill, state traffic) weigh: from step 2 on, two steps share a launch
     * when their chunks have the same size (their slots are then adjacent
     * rows of one buffer). Steps 0 and 1 stay alone: 0 needs no transfer and
     * 1 is the first to arrive. */
    const int pair_from = (even_rows && nranks >= 6) ? 2 : nranks;
    int n = 0;
    for (int s = 0; s < nranks; n++) {
        const int c = (s >= pair_from && s + 1 < nranks) ? 2 : 1;
        first_step[n] = s;
        step_count[n] = c;
        s += c;
    }
    return n;
}

/* ------------------------------------------------------------------------
 * Chunked attention with carried state
 * ------------------------------------------------------------------------ */

/* max_split: 2 lets a launch that fills the SMs badly split its keys in two. */
static int attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                           const uint16_t *k, const uint16_t *v, int ldkv,
                           int seq_q, int seq_k, int heads, float scale,
                           const int *key_mask, float *o_state, float *lse_state,
                           int first, int last, int max_split) {
    if (!require_device("attention_chunk")) return IRIS_B200_ENODEV;
    if (!q || !k || !v || seq_q < 0 || seq_k <= 0 || heads <= 0 || (last && !out) ||
        (!(first && last) && (!o_state || !lse_state))) {
        set_error(IRIS_B200_EINVAL, "attention_chunk", "bad argument");
        return IRIS_B200_EINVAL;
    }
    const void *o = out ? (const void *)out : (const void *)q;
    if (!sm100_supported(o, out ? ldo : 8, q, k, v, ldkv, heads, heads, 128, 0, scale) || ldq % 8 != 0 ||
        ((uintptr_t)o_state & 15) != 0) {
        set_error(IRIS_B200_EUNSUPPORTED, "attention_chunk", "arguments outside the tcgen05 kernel's domain");
        return IRIS_B200_EUNSUPPORTED;
    }
    if (seq_q == 0) return IRIS_B200_OK;
    int mode = first ? (last ? 0 : 1) : (last ? 3 : 2);
    return launch_attention_sm100(out, ldo, q, ldq, k, v, ldkv, seq_q, seq_k, heads, scale, key_mask, mode,
                                  o_state, lse_state, NULL, NULL, max_split);
}

extern "C" int iris_b200_attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                                         const uint16_t *k, const uint16_t *v, int ldkv,
                                         int seq_q, int seq_k, int heads, float scale,
                                         const int *key_mask, float *o_state, float *lse_state,
                                         int first, int last) {
    return attention_chunk(out, ldo, q, ldq, k, v, ldkv, seq_q, seq_k, heads, scale, key_mask, o_state, lse_state,
                           first, last, 2);
}

/* ------------------------------------------------------------------------
 * Ring sequence parallelism
 *
 * Rank r holds the query rows and the K / V rows of its token block. Step s
 * (s = 0 .. G-1) computes the attention of the local queries against the
 * chunk of rank (r - s) mod G and merges it into the carried state. The
 * chunk of step s is sent by its owner directly: at step s every rank sends
 * its own chunk to rank r + s and receives from rank r - s (NVSwitch gives
 * every pair full bandwidth, so nothing is relayed and no transfer waits
 * for a computation). All transfers are queued on a communication stream
 * when the call starts. Transport: the copy engines push the rows from the
 * caller's buffers into the consumer's slot (pools mapped through CUDA IPC)
 * and then write the call's sequence number into its arrival word, on
 * which the consumer's streams wait; NCCL send / recv with events when that
 * cannot be set up. NCCL also carries the set-up exchanges. A received
 * chunk lies in this GPU's memory before a kernel reads it.
 *
 * The heads are processed as two independent halves on two streams: a ring
 * step is a small problem (its CTAs fill the SMs about one and a half times),
 * and the CTAs of one half fill the SMs the tail of the other leaves idle.
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
typedef CUresult (*FnStreamValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

enum { kMaxRanks = 16, kHeadGroups = 2 };

struct Ring {
    void *dl;
    FnGetUniqueId get_id;
    FnCommInitRank init_rank;
    FnCommDestroy destroy;
    FnSendRecv send, recv;
    FnGroup group_start, group_end;
    FnErrStr err_str;
    FnAllGather all_gather;
    NcclComm comm;
    int rank, nranks;
    cudaStream_t comm_stream, aux_stream;
    cudaEvent_t received[kMaxRanks], packed, comm_done, join;
    void *buf[kMaxRanks];                 /* [0] local chunk, [s] chunk of step s */
    size_t buf_bytes[kMaxRanks];
    float *o_state[kHeadGroups], *lse_state[kHeadGroups];
    size_t o_bytes[kHeadGroups], lse_bytes[kHeadGroups];
    /* Copy-engine transport: chunks are pushed into the peers' slot pools
     * (mapped through CUDA IPC) by cudaMemcpyAsync, flow-controlled by
     * sequence numbers in device memory that streams wait on. */
    int ce;                               /* 0 not set up, 1 in use, -1 unavailable (NCCL send/recv instead) */
    FnStreamValue32 wait32, write32;
    char *pool;                           /* two sets (call parity) of nranks slots of slot_bytes: [s] step s */
    size_t slot_bytes;
    uint32_t *flags;                      /* arrive[kMaxRanks] | unused[kMaxRanks] | seq_words[8] */
    char *peer_pool[kMaxRanks];
    uint32_t *peer_flags[kMaxRanks];
    void *xchg;                           /* device staging of the handle exchange */
    uint32_t seq;
    /* IRIS_B200_RING_TRACE=1: device timeline of the last call, printed by ring_destroy() */
    int trace;                            /* -1 off, 1 on, 0 not looked up yet */
    cudaEvent_t t_start, t_push[kMaxRanks], t_step[kMaxRanks][2];
    int t_steps, t_pushes;
} ring = {};

enum { kFlagArrive = 0, kFlagSeq = 2 * kMaxRanks, kFlagWords = 2 * kMaxRanks + 8 };

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
    if (!ring.get_id || !ring.init_rank || !ring.destroy || !ring.send || !ring.recv || !ring.group_start ||
        !ring.group_end) {
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

bool grow(void **p, size_t *have, size_t need) {
    if (need <= *have) return true;
    if (*p) {
        cuda_ok(cudaDeviceSynchronize(), "sync");
        cuda_ok(cudaFree(*p), "free");
    }
    *p = NULL;
    *have = 0;
    if (cudaMalloc(p, need) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error(IRIS_B200_ENOMEM, "ring buffers", NULL);
        return false;
    }
    *have = need;
    return true;
}

/* Launches of the library go to g.stream; this redirects them for a scope. */
struct StreamScope {
    cudaStream_t saved;
    explicit StreamScope(cudaStream_t s) : saved(g.stream) { g.stream = s; }
    ~StreamScope() { g.stream = saved; }
};

}  // namespace


namespace {

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

void ce_free_pool(void) {
    if (ring.pool) cuda_ok(cudaFree(ring.pool), "free");
    ring.pool = NULL;
    ring.slot_bytes = 0;
}

/* All ranks have reached this point (an all-gather of a few bytes). */
bool ce_barrier(void) {
    if (!ring.xchg || !ring.all_gather) return false;
    char *dev = (char *)ring.xchg;
    return nccl_ok(ring.all_gather(dev + sizeof(IpcPair) * kMaxRanks, dev, 4, 1, ring.comm, g.stream), "ncclAllGather") &&
           cuda_ok(cudaStreamSynchronize(g.stream), "sync");
}

/* Collective: every rank calls it with the same slot size. Allocates (or
 * grows) the slot pool, exchanges the IPC handles through an NCCL all-gather
 * and maps the peers' pools and flag words. Returns false, with the NCCL
 * send/recv transport selected, when anything on the way is unavailable. */
bool ce_setup(size_t slot_bytes) {
    if (ring.ce < 0) return false;
    if (ring.ce == 1 && slot_bytes <= ring.slot_bytes) return true;
    const char *env = getenv("IRIS_B200_RING_TRANSPORT");
    const int G = ring.nranks;
    bool want = !(env && strcmp(env, "nccl") == 0) && ring.all_gather != NULL;
    if (want && !ring.wait32) {
        void *w = NULL, *wr = NULL;
        cudaDriverEntryPointQueryResult q1, q2;
        if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &w, cudaEnableDefault, &q1) != cudaSuccess ||
            cudaGetDriverEntryPoint("cuStreamWriteValue32", &wr, cudaEnableDefault, &q2) != cudaSuccess ||
            q1 != cudaDriverEntryPointSuccess || q2 != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            want = false;
        }
        ring.wait32 = (FnStreamValue32)w;
        ring.write32 = (FnStreamValue32)wr;
    }
    if (!want) {
        ring.ce = -1;
        return false;
    }
    /* Nobody may still be pushing into a pool that is about to go away. */
    cuda_ok(cudaDeviceSynchronize(), "sync");
    if (!ring.xchg && !cuda_ok(cudaMalloc(&ring.xchg, sizeof(IpcPair) * (kMaxRanks + 1)), "malloc")) return false;
    IpcPair *dev = (IpcPair *)ring.xchg;
    if (!ce_barrier()) return false;                /* every rank's pushes are complete */
    ce_close_peers();
    if (!ce_barrier()) return false;                /* every mapping of the old pools is gone */
    ce_free_pool();
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
    IpcPair mine, all[kMaxRanks];
    if (!cuda_ok(cudaIpcGetMemHandle(&mine.pool, ring.pool), "cudaIpcGetMemHandle") ||
        !cuda_ok(cudaIpcGetMemHandle(&mine.flags, ring.flags), "cudaIpcGetMemHandle") ||
        !cuda_ok(cudaMemcpy(dev + kMaxRanks, &mine, sizeof(mine), cudaMemcpyHostToDevice), "memcpy") ||
        !nccl_ok(ring.all_gather(dev + kMaxRanks, dev, sizeof(IpcPair), 1, ring.comm, g.stream), "ncclAllGather") ||
        !cuda_ok(cudaStreamSynchronize(g.stream), "sync") ||
        !cuda_ok(cudaMemcpy(all, dev, sizeof(IpcPair) * G, cudaMemcpyDeviceToHost), "memcpy"))
        return false;
    for (int r = 0; r < G; r++) {
        if (r == ring.rank) continue;
        void *pp = NULL, *pf = NULL;
        if (!cuda_ok(cudaIpcOpenMemHandle(&pp, all[r].pool, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle") ||
            !cuda_ok(cudaIpcOpenMemHandle(&pf, all[r].flags, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle"))
            return false;
        ring.peer_pool[r] = (char *)pp;
        ring.peer_flags[r] = (uint32_t *)pf;
    }
    ring.ce = 1;
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
    if (!cuda_ok(cudaStreamCreateWithFlags(&ring.comm_stream, cudaStreamNonBlocking), "stream create") ||
        !cuda_ok(cudaStreamCreateWithFlags(&ring.aux_stream, cudaStreamNonBlocking), "stream create"))
        return IRIS_B200_ECUDA;
    for (int i = 0; i < kMaxRanks; i++)
        cuda_ok(cudaEventCreateWithFlags(&ring.received[i], cudaEventDisableTiming), "event create");
    cuda_ok(cudaEventCreateWithFlags(&ring.packed, cudaEventDisableTiming), "event create");
    cuda_ok(cudaEventCreateWithFlags(&ring.comm_done, cudaEventDisableTiming), "event create");
    cuda_ok(cudaEventCreateWithFlags(&ring.join, cudaEventDisableTiming), "event create");
    return g.last_error;
}

extern "C" void iris_b200_ring_destroy(void) {
    if (!ring.comm) return;
    cuda_ok(cudaDeviceSynchronize(), "sync");
    if (ring.trace == 1 && ring.t_steps > 0) {
        /* Timeline of the last call, milliseconds after its start on the library's stream. */
        char line[1024];
        int n = snprintf(line, sizeof(line), "iris_b200 ring trace, rank %d:", ring.rank);
        float ms = 0.0f;
        for (int s = 1; s < ring.t_pushes && n < 900; s++)
            if (cudaEventElapsedTime(&ms, ring.t_start, ring.t_push[s]) == cudaSuccess)
                n += snprintf(line + n, sizeof(line) - n, " push%d=%.3f", s, ms);
        for (int i = 0; i < ring.t_steps && n < 900; i++) {
            float a = 0.0f, b = 0.0f;
            if (cudaEventElapsedTime(&a, ring.t_start, ring.t_step[i][0]) == cudaSuccess &&
                cudaEventElapsedTime(&b, ring.t_start, ring.t_step[i][1]) == cudaSuccess)
                n += snprintf(line + n, sizeof(line) - n, " launch%d=[%.3f,%.3f]", i, a, b);
        }
        fprintf(stderr, "%s\n", line);
        (void)cudaGetLastError();
    }
    ce_close_peers();
    if (ring.ce == 1) ce_barrier();
    ce_free_pool();
    if (ring.flags) cuda_ok(cudaFree(ring.flags), "free");
    if (ring.xchg) cuda_ok(cudaFree(ring.xchg), "free");
    ring.flags = NULL;
    ring.xchg = NULL;
    ring.ce = 0;
    ring.seq = 0;
    ring.destroy(ring.comm);
    ring.comm = NULL;
    for (int i = 0; i < kMaxRanks; i++) {
        if (ring.buf[i]) cuda_ok(cudaFree(ring.buf[i]), "free");
        ring.buf[i] = NULL;
        ring.buf_bytes[i] = 0;
        cuda_ok(cudaEventDestroy(ring.received[i]), "event destroy");
    }
    for (int i = 0; i < kHeadGroups; i++) {
        if (ring.o_state[i]) cuda_ok(cudaFree(ring.o_state[i]), "free");
        if (ring.lse_state[i]) cuda_ok(cudaFree(ring.lse_state[i]), "free");
        ring.o_state[i] = ring.lse_state[i] = NULL;
        ring.o_bytes[i] = ring.lse_bytes[i] = 0;
    }
    cuda_ok(cudaEventDestroy(ring.packed), "event destroy");
    cuda_ok(cudaEventDestroy(ring.comm_done), "event destroy");
    cuda_ok(cudaEventDestroy(ring.join), "event destroy");
    cuda_ok(cudaStreamDestroy(ring.comm_stream), "stream destroy");
    cuda_ok(cudaStreamDestroy(ring.aux_stream), "stream destroy");
}

/* rows_of[r]: token rows of rank r. q, k, v: this rank's rows, row stride
 * ldi. Chunk layout in the buffers: [rows, 2 * heads * 128] (K | V). */
extern "C" int iris_b200_ring_attention(uint16_t *out, int ldo,
                                        const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                        int ldi, const int *rows_of, int heads, float scale) {
    if (!require_device("ring_attention")) return IRIS_B200_ENODEV;
    if (!ring.comm || !rows_of || !out || !q || !k || !v || heads <= 0) {
        set_error(IRIS_B200_EINVAL, "ring_attention", "ring not initialised or bad argument");
        return IRIS_B200_EINVAL;
    }
    const int G = ring.nranks, me = ring.rank;
    const int rows = rows_of[me];
    const size_t width = (size_t)heads * 128;
    const int ngroups = (G > 1 && heads % kHeadGroups == 0) ? kHeadGroups : 1;
    const int hg = heads / ngroups;                         /* heads of one group */
    int max_rows = 0;
    for (int r = 0; r < G; r++) max_rows = rows_of[r] > max_rows ? rows_of[r] : max_rows;
    const size_t slot_bytes = ((size_t)max_rows * 2 * width * 2 + 255) & ~(size_t)255;

    /* Transport: pushes by the copy engines into IPC-mapped slot pools when
     * that can be set up, NCCL send/recv into private buffers otherwise. */
    const bool ce = G > 1 && ce_setup(slot_bytes);
    if (!ce && G > 1) {
        for (int s = 0; s < G; s++)
            if (!grow(&ring.buf[s], &ring.buf_bytes[s], slot_bytes)) return IRIS_B200_ENOMEM;
    }
    const uint32_t seq = ++ring.seq;
    /* Copy-engine slots come in two sets used by alternate calls. A peer
     * pushes the rows of call n + 1 only after its own call n, which waited
     * for this rank's push of call n, itself ordered after this rank's call
     * n - 1: the set of call n + 1 was last read here in call n - 1, so no
     * acknowledgement has to travel back. */
    const size_t set_off = ce ? (size_t)(seq & 1u) * G * ring.slot_bytes : 0;
    auto chunk = [&](int s) -> char * {
        return ce ? ring.pool + set_off + (size_t)s * ring.slot_bytes : (char *)ring.buf[s];
    };
    if (G > 1) {
        for (int i = 0; i < ngroups; i++)
            if (!grow((void **)&ring.o_state[i], &ring.o_bytes[i], (size_t)rows * hg * 128 * 4) ||
                !grow((void **)&ring.lse_state[i], &ring.lse_bytes[i], (size_t)rows * hg * 4))
                return IRIS_B200_ENOMEM;
    }
    uint32_t *seq_word = ce ? ring.flags + kFlagSeq + (seq & 7u) : NULL;
    const size_t my_bytes = (size_t)rows * 2 * width * 2;
    const size_t row_bytes = width * 2, slot_pitch = 2 * width * 2;      /* a slot row is K | V */

    /* Step 0 reads the local rows. The copy engines take them from the
     * caller's buffers as they are; NCCL wants them contiguous in slot 0. */
    const uint16_t *k0 = k, *v0 = v;
    int ld0 = ldi;
    if (ce) {
        /* Every earlier use of the sequence word is ordered before this
         * point on the library's stream. */
        if (!stream_value(ring.write32, g.stream, seq_word, seq, CU_STREAM_WRITE_VALUE_DEFAULT, "write seq"))
            return IRIS_B200_ECUDA;
    } else if (G > 1) {
        if (!cuda_ok(cudaMemcpy2DAsync(chunk(0), slot_pitch, k, (size_t)ldi * 2, row_bytes, rows,
                                       cudaMemcpyDeviceToDevice, g.stream), "pack K") ||
            !cuda_ok(cudaMemcpy2DAsync(chunk(0) + row_bytes, slot_pitch, v, (size_t)ldi * 2, row_bytes, rows,
                                       cudaMemcpyDeviceToDevice, g.stream), "pack V"))
            return IRIS_B200_ECUDA;
        k0 = (const uint16_t *)chunk(0);
        v0 = k0 + width;
        ld0 = (int)(2 * width);
    }
    cuda_ok(cudaEventRecord(ring.packed, g.stream), "event record");
    cuda_ok(cudaStreamWaitEvent(ring.comm_stream, ring.packed, 0), "stream wait");
    if (ring.trace == 0) {
        const char *env = getenv("IRIS_B200_RING_TRACE");
        ring.trace = env && env[0] == '1' ? 1 : -1;
        if (ring.trace == 1) {
            cudaEventCreate(&ring.t_start);
            for (int i = 0; i < kMaxRanks; i++) {
                cudaEventCreate(&ring.t_push[i]);
                cudaEventCreate(&ring.t_step[i][0]);
                cudaEventCreate(&ring.t_step[i][1]);
            }
        }
    }
    const bool trace = ring.trace == 1 && ce;
    if (trace) {
        cudaEventRecord(ring.t_start, g.stream);
        ring.t_steps = ring.t_pushes = 0;
    }

    /* All transfers, in step order on one stream: at step s this rank's rows
     * are wanted by rank me + s, which keeps them in its slot s. (Pushes on
     * two streams were measured to share one copy engine and run one after
     * the other anyway, 48 us per 26 MB, only no longer in the order the
     * steps need them.) */
    for (int s = 1; s < G; s++) {
        const int to = (me + s) % G, from = iris_b200_ring_source(me, s, G);
        if (ce) {
            cudaStream_t cs = ring.comm_stream;
            char *dst = ring.peer_pool[to] + set_off + (size_t)s * ring.slot_bytes;
            bool ok;
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
            if (!ok || !cuda_ok(cudaMemcpyAsync(ring.peer_flags[to] + kFlagArrive + s, seq_word, 4, cudaMemcpyDefault, cs),
                                "push flag"))
                return IRIS_B200_ECUDA;
            if (trace) {
                cudaEventRecord(ring.t_push[s], cs);
                ring.t_pushes = s + 1;
            }
        } else {
            if (!nccl_ok(ring.group_start(), "ncclGroupStart")) return IRIS_B200_ECOMM;
            bool ok = nccl_ok(ring.send(chunk(0), my_bytes, 1, to, ring.comm, ring.comm_stream), "ncclSend") &&
                      nccl_ok(ring.recv(chunk(s), (size_t)rows_of[from] * 2 * width * 2, 1, from, ring.comm,
                                        ring.comm_stream), "ncclRecv");
            if (!nccl_ok(ring.group_end(), "ncclGroupEnd") || !ok) return IRIS_B200_ECOMM;
            cuda_ok(cudaEventRecord(ring.received[s], ring.comm_stream), "event record");
        }
    }
    cuda_ok(cudaEventRecord(ring.comm_done, ring.comm_stream), "event record");

    /* Launch schedule: which steps share a launch (only chunks of one size
     * lying in adjacent slots can). */
    bool even = ce && ring.slot_bytes == my_bytes;
    for (int r = 0; r < G && even; r++) even = rows_of[r] == rows;
    int plan_first[kMaxRanks], plan_count[kMaxRanks];
    const int nlaunch = iris_b200_ring_plan(G, even ? 1 : 0, plan_first, plan_count);

    /* The head groups run side by side: group 0 on the library's stream,
     * group 1 on the auxiliary one, joined again before the call returns. */
    if (ngroups > 1) cuda_ok(cudaStreamWaitEvent(ring.aux_stream, ring.packed, 0), "stream wait");
    int rc = IRIS_B200_OK;
    for (int li = 0; li < nlaunch && rc == IRIS_B200_OK; li++) {
        const int s = plan_first[li], nsteps = plan_count[li];
        const int src = iris_b200_ring_source(me, s, G);
        const uint16_t *kc = s == 0 ? k0 : (const uint16_t *)chunk(s);
        const uint16_t *vc = s == 0 ? v0 : kc + width;
        const int ldc = s == 0 ? ld0 : (int)(2 * width);
        const int keys = nsteps > 1 ? nsteps * rows : rows_of[src];
        for (int grp = 0; grp < ngroups && rc == IRIS_B200_OK; grp++) {
            cudaStream_t st = grp == 0 ? g.stream : ring.aux_stream;
            for (int w = s; w < s + nsteps; w++) {
                if (w == 0) continue;
                if (ce) {
                    if (!stream_value(ring.wait32, st, ring.flags + kFlagArrive + w, seq, CU_STREAM_WAIT_VALUE_GEQ,
                                      "wait chunk"))
                        return IRIS_B200_ECUDA;
                } else {
                    cuda_ok(cudaStreamWaitEvent(st, ring.received[w], 0), "stream wait");
                }
            }
            StreamScope scope(st);
            const size_t col = (size_t)grp * hg * 128;
            if (trace && grp == 0) cudaEventRecord(ring.t_step[ring.t_steps][0], st);
            /* The head groups fill the SMs between them: no key split inside a launch. */
            rc = attention_chunk(out + col, ldo, q + col, ldi, kc + col, vc + col, ldc, rows, keys, hg, scale, NULL,
                                 ring.o_state[grp], ring.lse_state[grp], s == 0, s + nsteps == G, ngroups > 1 ? 1 : 2);
            if (trace && grp == 0) cudaEventRecord(ring.t_step[ring.t_steps++][1], st);
        }
    }
    if (ngroups > 1) {
        cuda_ok(cudaEventRecord(ring.join, ring.aux_stream), "event record");
        cuda_ok(cudaStreamWaitEvent(g.stream, ring.join, 0), "stream wait");
    }
    /* The transfers of the local rows must not outlive the call. */
    cuda_ok(cudaStreamWaitEvent(g.stream, ring.comm_done, 0), "stream wait");
    return rc != IRIS_B200_OK ? rc : g.last_error;
}
