/*
 * Multi-GPU decompositions of the joint attention (one process per GPU).
 *
 *  - head shards and the CFG split are pure index arithmetic: a rank runs the
 *    ordinary attention on its column slice, nothing is exchanged;
 *  - chunked attention: one launch sees a chunk of the keys and merges its
 *    result into a carried state (normalised fp32 output + log2-sum-exp per
 *    row), the building block of split-K and of the ring;
 *  - ring sequence parallelism: every rank keeps its query rows, the K/V
 *    chunks travel round the ring through NCCL send/recv on a second stream
 *    while the attention of the resident chunk runs. A received chunk lands
 *    in this GPU's own memory and is read from there by ordinary TMA loads.
 *
 * The reference has no multi-GPU code (iris_cuda.cu:122 always uses device
 * 0); these entry points are additions with no counterpart there.
 *
 * NCCL is loaded at run time (dlopen) so that the single-GPU library has no
 * link-time dependency on it.
 */
#include "common.cuh"

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

/* ------------------------------------------------------------------------
 * Chunked attention with carried state
 * ------------------------------------------------------------------------ */

extern "C" int iris_b200_attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                                         const uint16_t *k, const uint16_t *v, int ldkv,
                                         int seq_q, int seq_k, int heads, float scale,
                                         const int *key_mask, float *o_state, float *lse_state,
                                         int first, int last) {
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
                                  o_state, lse_state, NULL, NULL);
}

/* ------------------------------------------------------------------------
 * NCCL ring
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

struct Ring {
    void *dl;
    FnGetUniqueId get_id;
    FnCommInitRank init_rank;
    FnCommDestroy destroy;
    FnSendRecv send, recv;
    FnGroup group_start, group_end;
    FnErrStr err_str;
    NcclComm comm;
    int rank, nranks;
    cudaStream_t comm_stream;
    cudaEvent_t computed[2], received[2], packed;
    void *buf[2];
    size_t buf_bytes[2];
    float *o_state, *lse_state;
    size_t o_bytes, lse_bytes;
} ring = {};

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
        cuda_ok(cudaStreamSynchronize(g.stream), "sync");
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
    if (!id128 || nranks < 1 || rank < 0 || rank >= nranks || ring.comm) return IRIS_B200_EINVAL;
    if (!nccl_load()) return IRIS_B200_ECOMM;
    NcclId id;
    memcpy(&id, id128, sizeof(id));
    if (!nccl_ok(ring.init_rank(&ring.comm, nranks, id, rank), "ncclCommInitRank")) {
        ring.comm = NULL;
        return IRIS_B200_ECOMM;
    }
    ring.rank = rank;
    ring.nranks = nranks;
    if (!cuda_ok(cudaStreamCreateWithFlags(&ring.comm_stream, cudaStreamNonBlocking), "stream create"))
        return IRIS_B200_ECUDA;
    for (int i = 0; i < 2; i++) {
        cuda_ok(cudaEventCreateWithFlags(&ring.computed[i], cudaEventDisableTiming), "event create");
        cuda_ok(cudaEventCreateWithFlags(&ring.received[i], cudaEventDisableTiming), "event create");
    }
    cuda_ok(cudaEventCreateWithFlags(&ring.packed, cudaEventDisableTiming), "event create");
    return g.last_error;
}

extern "C" void iris_b200_ring_destroy(void) {
    if (!ring.comm) return;
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
    cuda_ok(cudaStreamSynchronize(ring.comm_stream), "sync");
    ring.destroy(ring.comm);
    ring.comm = NULL;
    for (int i = 0; i < 2; i++) {
        if (ring.buf[i]) cuda_ok(cudaFree(ring.buf[i]), "free");
        ring.buf[i] = NULL;
        ring.buf_bytes[i] = 0;
        cuda_ok(cudaEventDestroy(ring.computed[i]), "event destroy");
        cuda_ok(cudaEventDestroy(ring.received[i]), "event destroy");
    }
    cuda_ok(cudaEventDestroy(ring.packed), "event destroy");
    if (ring.o_state) cuda_ok(cudaFree(ring.o_state), "free");
    if (ring.lse_state) cuda_ok(cudaFree(ring.lse_state), "free");
    ring.o_state = ring.lse_state = NULL;
    ring.o_bytes = ring.lse_bytes = 0;
    cuda_ok(cudaStreamDestroy(ring.comm_stream), "stream destroy");
}

/* Every rank holds `rows` query rows and the K / V rows of the same tokens
 * (rows may differ per rank: rows_of[r], r = 0..nranks-1). Step s computes
 * the attention of the local queries against the chunk that started on rank
 * (rank - s) mod nranks while that chunk is already on its way to rank + 1.
 * Chunk layout in the ring buffers: [rows, 2 * heads * 128] (K | V). */
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
    int max_rows = 0;
    for (int r = 0; r < G; r++) max_rows = rows_of[r] > max_rows ? rows_of[r] : max_rows;
    const size_t chunk_bytes = (size_t)max_rows * 2 * width * 2;
    for (int i = 0; i < 2; i++)
        if (!grow(&ring.buf[i], &ring.buf_bytes[i], chunk_bytes)) return IRIS_B200_ENOMEM;
    if (G > 1) {
        if (!grow((void **)&ring.o_state, &ring.o_bytes, (size_t)rows * width * 4) ||
            !grow((void **)&ring.lse_state, &ring.lse_bytes, (size_t)rows * heads * 4))
            return IRIS_B200_ENOMEM;
    }
    /* The local chunk goes into buffer 0 as [rows, K | V]. */
    if (!cuda_ok(cudaMemcpy2DAsync(ring.buf[0], 2 * width * 2, k, (size_t)ldi * 2, width * 2, rows,
                                   cudaMemcpyDeviceToDevice, g.stream), "pack K") ||
        !cuda_ok(cudaMemcpy2DAsync((char *)ring.buf[0] + width * 2, 2 * width * 2, v, (size_t)ldi * 2, width * 2,
                                   rows, cudaMemcpyDeviceToDevice, g.stream), "pack V"))
        return IRIS_B200_ECUDA;
    cuda_ok(cudaEventRecord(ring.packed, g.stream), "event record");
    cuda_ok(cudaStreamWaitEvent(ring.comm_stream, ring.packed, 0), "stream wait");

    /* IRIS_B200_RING_TRACE=1: per-step device times of the two streams on stderr. */
    static int trace = -1;
    if (trace < 0) {
        const char *e = getenv("IRIS_B200_RING_TRACE");
        trace = e && e[0] == '1';
    }
    enum { kMaxTrace = 64 };
    static cudaEvent_t tev[kMaxTrace][4];
    static int tev_made = 0;
    if (trace && !tev_made) {
        for (int i = 0; i < kMaxTrace; i++)
            for (int j = 0; j < 4; j++) cudaEventCreate(&tev[i][j]);
        tev_made = 1;
    }
    const int next = (me + 1) % G, prev = (me + G - 1) % G;
    for (int s = 0; s < G; s++) {
        const int cur = s & 1, nxt = cur ^ 1;
        const int src = iris_b200_ring_source(me, s, G);           /* owner of the resident chunk */
        if (s + 1 < G) {
            /* Forward the resident chunk, receive the next one. The target
             * buffer was last read by the attention of step s - 1. */
            if (s >= 1) cuda_ok(cudaStreamWaitEvent(ring.comm_stream, ring.computed[nxt], 0), "stream wait");
            const int incoming = iris_b200_ring_source(me, s + 1, G);
            if (trace && s < kMaxTrace) cudaEventRecord(tev[s][0], ring.comm_stream);
            if (!nccl_ok(ring.group_start(), "ncclGroupStart")) return IRIS_B200_ECOMM;
            bool ok = nccl_ok(ring.send(ring.buf[cur], (size_t)rows_of[src] * 2 * width * 2, 1, next, ring.comm,
                                        ring.comm_stream), "ncclSend") &&
                      nccl_ok(ring.recv(ring.buf[nxt], (size_t)rows_of[incoming] * 2 * width * 2, 1, prev,
                                        ring.comm, ring.comm_stream), "ncclRecv");
            if (!nccl_ok(ring.group_end(), "ncclGroupEnd") || !ok) return IRIS_B200_ECOMM;
            cuda_ok(cudaEventRecord(ring.received[nxt], ring.comm_stream), "event record");
            if (trace && s < kMaxTrace) cudaEventRecord(tev[s][1], ring.comm_stream);
        }
        if (s >= 1) cuda_ok(cudaStreamWaitEvent(g.stream, ring.received[cur], 0), "stream wait");
        const uint16_t *kc = (const uint16_t *)ring.buf[cur];
        if (trace && s < kMaxTrace) cudaEventRecord(tev[s][2], g.stream);
        int rc = iris_b200_attention_chunk(out, ldo, q, ldi, kc, kc + width, (int)(2 * width), rows, rows_of[src],
                                           heads, scale, NULL, ring.o_state, ring.lse_state, s == 0, s == G - 1);
        if (rc != IRIS_B200_OK) return rc;
        cuda_ok(cudaEventRecord(ring.computed[cur], g.stream), "event record");
        if (trace && s < kMaxTrace) cudaEventRecord(tev[s][3], g.stream);
    }
    /* The send of the last forwarded chunk must not outlive the call. */
    cuda_ok(cudaEventRecord(ring.packed, ring.comm_stream), "event record");
    cuda_ok(cudaStreamWaitEvent(g.stream, ring.packed, 0), "stream wait");
    if (trace) {
        cudaStreamSynchronize(g.stream);
        for (int s = 0; s < G && s < kMaxTrace; s++) {
            float c0 = 0, c1 = 0, k0 = 0, k1 = 0;
            if (s + 1 < G) {
                cudaEventElapsedTime(&c0, tev[0][2], tev[s][0]);
                cudaEventElapsedTime(&c1, tev[0][2], tev[s][1]);
            }
            cudaEventElapsedTime(&k0, tev[0][2], tev[s][2]);
            cudaEventElapsedTime(&k1, tev[0][2], tev[s][3]);
            fprintf(stderr, "ring rank %d step %d: comm [%.3f, %.3f] ms  attention [%.3f, %.3f] ms\n", me, s, c0, c1, k0, k1);
        }
    }
    return g.last_error;
}
