/*
 * Joint attention for sm_100a: TMA loads, tcgen05 MMAs accumulating in
 * tensor memory, online softmax with one thread per query row.
 *
 * Takes the argument domain of the transformer blocks (the reference's own
 * fast-path test, iris_cuda.cu:884-886, tightened to what TMA needs):
 * head_dim 128, heads == kv_heads, non-causal, optional key mask, bf16
 * [seq, heads*128] views with 16-byte aligned bases and ldi % 8 == 0.
 *
 * Work decomposition
 *   A work item is 256 consecutive queries of one head, as two 128-row
 *   tiles, against a run of key tiles of 128. The grid is persistent (one CTA
 *   per SM at most). The CTAs draw items from one list in order (an atomic
 *   counter; the producer warp fetches the next index while the current item
 *   runs and hands it to the other warps through shared memory), so a CTA
 *   that was held up simply takes fewer items. Items are head-major: the
 *   CTAs working at the same time share the K/V of a few heads through L2.
 *   When the query blocks fill the SMs badly, or the keys arrive over time,
 *   the keys are cut into up to eight parts; the list then holds part 0 of
 *   every query block, then part 1, ...; the parts of a block leave their
 *   unnormalised results in scratch and whichever finishes last merges them.
 *
 * Keys
 *   The key rows are a sequence of sources: runs of rows inside one of two
 *   K/V views (two pairs of tensor maps), e.g. the caller's own rows followed
 *   by the slots other GPUs have copied their rows into. A source may be
 *   guarded by arrival words in device memory: before the first load of a
 *   tile the producer waits (bounded) until the words covering its rows have
 *   reached the call's sequence number. Every load reads this GPU's memory.
 *
 * Warps (384 threads)
 *   0-3   softmax of query tile 0: thread r owns row r of S / P / O
 *   4-7   softmax of query tile 1
 *   8     scheduler and TMA producer (one lane): Q per item, then K0 V0 K1
 *         V1 ... through a ring of 32 KB slots guarded by full / empty
 *         mbarriers
 *   9     MMA issuer (whole warp, one elected lane issues), owner of the
 *         TMEM allocation
 *   10-11 idle: they complete the third warpgroup, which gives most of its
 *         registers to the softmax warpgroups (setmaxnreg)
 *
 * Tensor memory (512 columns x 128 lanes, fp32)
 *   [  0,128) S0   [128,256) S1   [256,384) O0   [384,512) O1
 *   P_t (bf16, 64 columns) overwrites the first half of S_t: a softmax
 *   thread has read its whole S row before it stores P.
 *
 * MMA issue order per key tile j (all from one thread, executed in order;
 * each PV in two halves of 64 keys as the softmax hands them over):
 *   PV0(j)  QK0(j+1)  PV1(j)  QK1(j+1)
 *   S_t = Q_t K^T : both operands from shared memory, K-major, 128B swizzle
 *   O_t += P_t V  : P from tensor memory, V from shared memory, MN-major
 *   While the tensor pipe works for tile t, the softmax warpgroup of the
 *   other tile turns its S into P, so the two overlap.
 *
 * Online softmax (base 2, scale * log2(e) folded into one FMA per score):
 *   the reference value m of a row only moves when the row maximum grows by
 *   more than 8 (a factor 256), so the O rescale in tensor memory is rare;
 *   P <= 256 keeps full precision in bf16 and fp32. P is rounded to bf16 for
 *   the MMA while the row sum keeps the unrounded value, as the reference
 *   kernel does (iris_cuda.cu:819-831). Masked and out-of-range keys score
 *   -inf; a row without any valid key yields zeros (iris_cuda.cu:811, :853).
 *
 * Output: accumulator rows go through a per-warp shared-memory staging area
 * so that global memory sees whole 128-byte segments of a row.
 *
 * Every wait (mbarriers, the other parts of a key split, arrival words) is
 * bounded in time (a launch parameter, one second unless the host sets
 * another): when the limit passes the CTA records where in the device status
 * word, raises a CTA-wide abort flag, drains what it has in flight (again
 * bounded), frees its tensor memory and returns. Every load is a TMA copy
 * issued by and for one CTA.
 */
#include "common.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "kernels.h"
#include "tc_ptx.cuh"
#include <math.h>

namespace iris_b200 {

namespace sm100 {

static constexpr int kTileQ = 128;            /* rows of one query tile / MMA M */
static constexpr int kTileK = 128;            /* keys per tile / MMA N of S */
static constexpr int kHeadDim = 128;
static constexpr int kStages = 4;             /* K / V ring slots */
static constexpr int kHalfBytes = 128 * 64 * 2;         /* one [128 x 64] bf16 swizzled box */
static constexpr int kTileBytes = 2 * kHalfBytes;       /* one [128 x 128] bf16 operand */
static constexpr int kThreads = 384;
static constexpr int kSmemQ = 0;
static constexpr int kSmemKV = 2 * kTileBytes;
static constexpr int kSmemStage = kSmemKV + kStages * kTileBytes;   /* output staging: 8 warps x 4 KB */
static constexpr int kSmemBar = kSmemStage + 8 * 4096;
static constexpr int kSmemBytes = kSmemBar + 256 + 1024;   /* + barriers + alignment slack */
static constexpr float kRescaleThreshold = 8.0f;
static constexpr int kRegsSoftmax = 216, kRegsOther = 72;   /* 2 * 224 + 56 <= 512 */
static constexpr int kMaxSources = AttnArgs::kMaxSources;
static constexpr int kMaxParts = AttnArgs::kMaxParts;
/* Shared memory descriptor fields, in 16-byte units */
static constexpr uint32_t kQkSbo = 1024 / 16;          /* 8 rows of 128 B */
static constexpr uint32_t kVLbo = kHalfBytes / 16;     /* next 64-dim half */
static constexpr uint32_t kVSbo = 1024 / 16;           /* next 8 keys */

/* mbarrier slots inside the barrier block (8 bytes each) */
enum {
    BAR_Q_FULL = 0,
    BAR_KV_FULL = 1,                      /* kStages */
    BAR_KV_EMPTY = BAR_KV_FULL + kStages, /* kStages */
    BAR_S_FULL = BAR_KV_EMPTY + kStages,  /* 2 */
    BAR_P_FULL = BAR_S_FULL + 2,          /* 4: [tile][half of the key tile] */
    BAR_O_DONE = BAR_P_FULL + 4,          /* 2 */
    BAR_Q_EMPTY = BAR_O_DONE + 2,         /* the QK products of a work item are complete */
    BAR_DRAIN,
    BAR_SCHED_FULL,                       /* 2: the index of work item n (slot n & 1) is published */
    BAR_SCHED_EMPTY = BAR_SCHED_FULL + 2, /* 2: every consumer warp has read it */
    BAR_COUNT = BAR_SCHED_EMPTY + 2
};
static constexpr int kSmemTmemPtr = BAR_COUNT * 8;      /* u32 */
static constexpr int kSmemAbort = kSmemTmemPtr + 4;     /* u32 */
static constexpr int kSmemSched = kSmemAbort + 4;       /* int [2] */
static_assert(kSmemSched + 8 <= 256, "barrier block");
static constexpr int kSchedConsumers = 9;               /* the MMA warp and the eight softmax warps */

/* A run of key rows inside one of the two K/V views. */
struct KeySource {
    int tile0;          /* first key tile (over all sources) */
    int row0;           /* first row inside the view */
    int rows;           /* keys */
    int view;           /* 0 / 1: which pair of tensor maps */
    int arrive;         /* index of the first arrival word guarding the rows, -1: none */
    int rows_per_word;  /* rows guarded by one word (consecutive words follow) */
};

struct Params {
    uint16_t *out;
    int ldo;
    int seq_q, heads;
    int nqblk;                 /* 256-row query blocks per head */
    int nq;                    /* query blocks over all heads */
    int items;                 /* work items: nq * nparts */
    int nkv;                   /* 128-key tiles over all sources */
    /* Key split: part i of a query block covers the tiles [part_tile[i],
     * part_tile[i + 1]); whichever part finishes last merges the others. */
    int nparts;
    int part_tile[kMaxParts + 1];
    int nsrc;
    KeySource src[kMaxSources];
    const uint32_t *arrive;    /* arrival words, or NULL */
    uint32_t arrive_seq;       /* a word has arrived when (int)(word - arrive_seq) >= 0 */
    float *part_o;             /* [nq, nparts - 1, 256, 128] fp32 unnormalised O of the parts that finished early */
    float2 *part_ml;           /* [nq, nparts - 1, 256] their (row maximum, row sum) */
    unsigned int *tickets;     /* [nq, 8 warps, 2]: arrivals, partials written; zero between launches */
    unsigned int *sched;       /* [0] next work item, [1] CTAs that are through; zero between launches; NULL: CTA b
                                  takes the items b, b + gridDim.x, ... */
    float scale_log2;
    const uint32_t *mask_bits; /* packed key mask, bit j of word j/32, or NULL (single source only) */
    unsigned int *status;      /* [0] flag, [1] site, [2] block, [3] aux */
    unsigned long long wait_ns; /* limit of every wait */
    int view_rows[2];          /* rows of the two K/V views (self-checks) */
    int part_cap, ticket_cap;  /* 256-row partials / query blocks the scratch has room for (self-checks) */
    /* state carried across key chunks (split-K over several launches), or NULL */
    float *o_acc;              /* [seq_q, heads*128] fp32, normalised partial output */
    float *lse_acc;            /* [heads, seq_q] fp32, log2-sum-exp of the keys seen so far */
    int acc_mode;              /* 0: single pass; 1: first chunk (write state); 2: merge into state;
                                  3: merge with the state and write the final bf16 output */
};

/* ---------------- bounded waits ---------------- */

struct Ctx {
    uint32_t bars;                  /* shared address of the barrier block */
    volatile uint32_t *abort_flag;  /* generic pointer to the CTA abort word */
    unsigned int *status;
    unsigned long long wait_ns;
};

/* A wait ran out: raise the CTA's abort flag and record the first such event
 * of the launch in the device status word. */
__device__ __forceinline__ void give_up(const Ctx &c, int site, unsigned aux) {
    *c.abort_flag = 1u;
    if (atomicCAS(c.status, 0u, 1u) == 0u) {
        c.status[1] = (unsigned)site;
        c.status[2] = blockIdx.x;
        c.status[3] = aux;
    }
}

/* Self-checks of the -DIRIS_B200_CHECK build (tile and slot indices, scratch
 * capacities, rows handed to TMA): a violated check never traps; it records
 * the first site in words 4-7 of the status word, which
 * iris_b200_check_device_status() reports as IRIS_B200_ECHECK, and the access
 * goes ahead only where it is harmless. Compiled out of the product build. */
#ifdef IRIS_B200_CHECK
__device__ __noinline__ void check_failed(unsigned int *status, int site, unsigned aux) {
    if (atomicCAS(status + 4, 0u, 1u) == 0u) {
        status[5] = (unsigned)site;
        status[6] = blockIdx.x;
        status[7] = aux;
    }
}
#define IRIS_CHECK(status, cond, site, aux) \
    do {                                     \
        if (!(cond)) check_failed((status), (site), (unsigned)(aux)); \
    } while (0)
#else
#define IRIS_CHECK(status, cond, site, aux) ((void)0)
#endif

/* Bounded wait. Returns false when the CTA is aborting. `site` identifies
 * the caller in the status word. */
__device__ __forceinline__ bool mbar_wait_slow(const Ctx &c, uint32_t bar, uint32_t parity, int site) {
    unsigned long long t0 = global_ns();
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 63u) {
            if (*c.abort_flag) return false;
            if (global_ns() - t0 > c.wait_ns || spin > (1u << 26)) {
                give_up(c, site, parity);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(const Ctx &c, int idx, uint32_t parity, int site) {
    uint32_t bar = c.bars + idx * 8;
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(c, bar, parity, site);
}

/* Bounded wait for a 32-bit word in global memory that somebody else (another
 * CTA, a copy engine, another GPU) advances to at least `target`. */
__device__ __forceinline__ bool word_reached(const uint32_t *word, uint32_t target) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
    return (int32_t)(v - target) >= 0;
}
__device__ __forceinline__ bool word_wait(const Ctx &c, const uint32_t *word, uint32_t target, int site, unsigned aux) {
    if (word_reached(word, target)) return true;
    unsigned long long t0 = global_ns();
    for (uint32_t spin = 0;; spin++) {
        if (word_reached(word, target)) return true;
        if ((spin & 7u) == 7u) {
            if (*c.abort_flag) return false;
            if (global_ns() - t0 > c.wait_ns || spin > (1u << 26)) {
                give_up(c, site, aux);
                return false;
            }
            __nanosleep(100);
        }
    }
}

/* Instruction descriptor, kind::f16: fp32 accumulate, bf16 operands,
 * M = 128, N = 128; bit 16 selects an MN-major B operand. */
static constexpr uint32_t kIdescBase = idesc_bf16(128, 128);
static constexpr uint32_t kIdescQK = kIdescBase;
static constexpr uint32_t kIdescPV = kIdescBase | (1u << 16);

/* ---------------- work items ---------------- */

/* Position in the K/V ring: tiles are consumed in load order K0 V0 K1 V1 ... */
struct Ring {
    int slot;
    uint32_t phase;
    __device__ __forceinline__ void next() {
        if (++slot == kStages) {
            slot = 0;
            phase ^= 1u;
        }
    }
};

/* A work item is one part of the keys for one 256-row query block of one
 * head. The list is part-major: item = part * nq + query block. */
struct Item {
    int qitem;          /* query block index over all heads */
    int head, q0, ntq;
    int j0, nj;         /* first key tile and number of key tiles */
};
__device__ __forceinline__ Item item_of(const Params &p, int item) {
    Item w;
    const int part = item / p.nq;
    w.qitem = item - part * p.nq;
    w.head = w.qitem / p.nqblk;
    w.q0 = (w.qitem - w.head * p.nqblk) * 2 * kTileQ;
    w.ntq = (p.seq_q - w.q0 > kTileQ) ? 2 : 1;
    w.j0 = p.part_tile[part];
    w.nj = p.part_tile[part + 1] - w.j0;
    return w;
}

/* Source that holds key tile j (sources are few: a linear walk). */
__device__ __forceinline__ int source_of(const Params &p, int j) {
    int s = 0;
    while (s + 1 < p.nsrc && p.src[s + 1].tile0 <= j) s++;
    return s;
}
/* Keys of tile j that exist, given its source. */
__device__ __forceinline__ int tile_keys(const KeySource &s, int j) {
    const int left = s.rows - (j - s.tile0) * kTileK;
    return left < kTileK ? left : kTileK;
}

/* The work list as seen by the warps that do not fetch from it: item n of
 * this CTA is published in slot n & 1 of a two-entry mailbox. Returns the
 * item index, -1 at the end of the list, -2 when the CTA is aborting. */
__device__ __forceinline__ int sched_get(const Ctx &c, const int *mail, int n, int site) {
    const int slot = n & 1;
    if (!__all_sync(0xffffffffu, mbar_wait(c, BAR_SCHED_FULL + slot, (n >> 1) & 1u, site))) return -2;
    const int item = mail[slot];
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(c.bars + (BAR_SCHED_EMPTY + slot) * 8);
    return item;
}

__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    return ((uint64_t)hi << 32) | lo;
}

/* ---------------- roles ---------------- */

struct Maps {
    const CUtensorMap *q, *k[2], *v[2];
};

__device__ __forceinline__ void producer(const Ctx &c, const Params &p, const Maps &m, uint32_t smem, volatile int *mail) {
    int issued = 0;
    Ring r = {0, 0u};
    bool ok = true;
    uint32_t arrived = 0;                   /* arrival words seen at their target value */

    /* Next index of the work list, and its publication as item n of this CTA. */
    auto take = [&](int n) -> int {
        const int item = p.sched ? (int)atomicAdd(p.sched, 1u) : (int)(blockIdx.x + (unsigned)n * gridDim.x);
        return item < p.items ? item : -1;
    };
    auto publish = [&](int n, int item) -> bool {
        const int slot = n & 1;
        /* The slot held item n - 2, which every consumer has read long ago. */
        if (n >= 2 && !mbar_wait(c, BAR_SCHED_EMPTY + slot, ((n >> 1) - 1) & 1u, 120 + slot)) return false;
        mail[slot] = item;
        mbar_arrive(c.bars + (BAR_SCHED_FULL + slot) * 8);
        return true;
    };

    int cur = take(0);
    ok = publish(0, cur);
    for (int n = 0; ok && cur >= 0; n++) {
        const Item w = item_of(p, cur);
        const int col = w.head * kHeadDim;
        IRIS_CHECK(c.status, cur < p.items && w.head < p.heads && w.q0 < p.seq_q && w.nj >= 1 && w.j0 >= 0 &&
                   w.j0 + w.nj <= p.nkv, 900, cur);
        /* The Q tiles are replaced once every QK product of the previous item is done. */
        if (n > 0 && !mbar_wait(c, BAR_Q_EMPTY, (n - 1) & 1, 110)) break;
        mbar_expect_tx(c.bars + BAR_Q_FULL * 8, w.ntq * kTileBytes);
        for (int t = 0; t < w.ntq; t++)
            for (int half = 0; half < 2; half++)
                tma_load_2d(smem + kSmemQ + t * kTileBytes + half * kHalfBytes, m.q, col + half * 64,
                            w.q0 + t * kTileQ, c.bars + BAR_Q_FULL * 8);
        int si = source_of(p, w.j0);
        int next = -1;
        bool fetched = false;
        for (int it = 0; it < 2 * w.nj; it++, issued++, r.next()) {
            /* The next item is fetched once the first tiles of this one are on
             * their way: the round trip of the atomic hides behind them. */
            if (!fetched && it >= 4) {
                next = take(n + 1);
                fetched = true;
                if (!(ok = publish(n + 1, next))) break;
            }
            const int j = w.j0 + (it >> 1);
            if (!(it & 1)) {
                while (si + 1 < p.nsrc && p.src[si + 1].tile0 <= j) si++;
                const KeySource &s = p.src[si];
                if (s.arrive >= 0) {
                    /* Rows of this tile inside the source, and the words that guard them. */
                    const int a = (j - s.tile0) * kTileK;
                    const int b = (a + kTileK < s.rows ? a + kTileK : s.rows) - 1;
                    for (int wd = s.arrive + a / s.rows_per_word; ok && wd <= s.arrive + b / s.rows_per_word; wd++) {
                        if ((arrived >> (wd & 31)) & 1u) continue;
                        ok = word_wait(c, p.arrive + wd, p.arrive_seq, 130, (unsigned)wd);
                        arrived |= 1u << (wd & 31);
                        /* The rows were written by a copy engine or another GPU; the
                         * loads below go through the asynchronous proxy. */
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    }
                    if (!ok) break;
                }
            }
            /* A slot is refilled once the MMAs that read its previous content are done. */
            if (issued >= kStages && !mbar_wait(c, BAR_KV_EMPTY + r.slot, r.phase ^ 1u, 100 + r.slot)) {
                ok = false;
                break;
            }
            const KeySource &s = p.src[si];
            IRIS_CHECK(c.status, si < p.nsrc && j >= s.tile0 && (j - s.tile0) * kTileK < s.rows &&
                       s.row0 + (j - s.tile0) * kTileK < p.view_rows[s.view] && r.slot < kStages, 901, j);
            uint32_t full = c.bars + (BAR_KV_FULL + r.slot) * 8;
            mbar_expect_tx(full, kTileBytes);
            const CUtensorMap *map = (it & 1) ? m.v[s.view] : m.k[s.view];
            for (int half = 0; half < 2; half++)
                tma_load_2d(smem + kSmemKV + r.slot * kTileBytes + half * kHalfBytes, map, col + half * 64,
                            s.row0 + (j - s.tile0) * kTileK, full);
        }
        if (ok && !fetched) {
            next = take(n + 1);
            ok = publish(n + 1, next);
        }
        cur = next;
    }
    if (*c.abort_flag) {
        /* Nobody may be consuming any more: wait for the copies still in flight. */
        for (int it = issued > kStages ? issued - kStages : 0; it < issued; it++)
            mbar_wait(c, BAR_KV_FULL + it % kStages, (it / kStages) & 1, 190);
    }
}

__device__ __forceinline__ void mma_issuer(const Ctx &c, const Params &p, uint32_t smem, uint32_t tmem, const int *mail) {
    /* Descriptor words that never change: the high word (stride offset,
     * version, swizzle mode) per operand kind, and the low word of each
     * tile base (start address and leading offset, 16-byte units). A k-step
     * only adds a constant to the low word. */
    const uint32_t hi_qk = (uint32_t)(make_desc(0, 0, kQkSbo) >> 32);
    const uint32_t hi_v = (uint32_t)(make_desc(0, 0, kVSbo) >> 32);
    const uint32_t lo_q0 = (uint32_t)make_desc(smem + kSmemQ, 1, 0);
    const uint32_t lo_k0 = (uint32_t)make_desc(smem + kSmemKV, 1, 0);
    const uint32_t lo_v0 = (uint32_t)make_desc(smem + kSmemKV, kVLbo, 0);
    const bool leader = elect_one();        /* the whole warp runs this code, one lane issues */
    bool ok = true;

    auto issue_qk = [&](int t, int slot) {
        const uint32_t lo_q = lo_q0 + t * (kTileBytes >> 4), lo_k = lo_k0 + slot * (kTileBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ks++) {
            const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
            if (leader)
                mma_ss(tmem + t * 128, desc64(lo_q + off, hi_qk), desc64(lo_k + off, hi_qk), kIdescQK, ks > 0);
        }
        if (leader) tc_commit(c.bars + (BAR_S_FULL + t) * 8);
    };
    /* Half h of the PV product of a key tile: keys [64 h, 64 h + 64). */
    auto issue_pv = [&](int t, int h, int slot, bool first) {
        const uint32_t lo_v = lo_v0 + slot * (kTileBytes >> 4) + h * (64 * 128 >> 4);
        const uint32_t tp = tmem + t * 128 + h * 32, to = tmem + 256 + t * 128;
        if (first && h == 0) {
#pragma unroll
            for (int ks = 0; ks < 4; ks++)
                if (leader) mma_ts(to, tp + ks * 8, desc64(lo_v + ks * (16 * 128 >> 4), hi_v), kIdescPV, ks > 0);
        } else {
#pragma unroll
            for (int ks = 0; ks < 4; ks++)
                if (leader) mma_ts(to, tp + ks * 8, desc64(lo_v + ks * (16 * 128 >> 4), hi_v), kIdescPV, 1);
        }
        if (h == 1 && leader) tc_commit(c.bars + (BAR_O_DONE + t) * 8);
    };

    Ring r = {0, 0u};
    uint32_t seen[2] = {0u, 0u};            /* key tiles of query tile t so far, over all items */
    for (int n = 0; ok; n++) {
        const int item = sched_get(c, mail, n, 240);
        if (item < 0) {
            ok = item == -1;
            break;
        }
        const Item w = item_of(p, item);
        const int ntq = w.ntq, nkv = w.nj;
        IRIS_CHECK(c.status, item < p.items && (ntq == 1 || ntq == 2) && nkv >= 1 && r.slot < kStages, 910, item);
        ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_Q_FULL, n & 1, 200) && mbar_wait(c, BAR_KV_FULL + r.slot, r.phase, 201));
        if (!ok) break;
        tc_fence_after();
        /* S of tile t is free: the last PV of the previous item, issued
         * before, read P from it, and the tensor pipe keeps the order. */
        for (int t = 0; t < ntq; t++) issue_qk(t, r.slot);
        if (leader) {
            tc_commit(c.bars + (BAR_KV_EMPTY + r.slot) * 8);
            if (nkv == 1) tc_commit(c.bars + BAR_Q_EMPTY * 8);
        }
        r.next();
        for (int j = 0; ok && j < nkv; j++) {
            const Ring rv = r;              /* V_j */
            r.next();
            const Ring rk = r;              /* K_{j+1}, when there is one */
            const bool more = j + 1 < nkv;
            if (more) r.next();
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_KV_FULL + rv.slot, rv.phase, 210)))) break;
            for (int t = 0; t < ntq; t++) {
                const uint32_t par = (seen[t] + j) & 1u;
                /* The first 64 keys' P arrives while the softmax is still busy
                 * with the other 64: their PV runs under it. (With j == 0 the
                 * softmax warps have also read the previous item's O by now.) */
                if (!(ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_P_FULL + 2 * t, par, 220 + t)))) break;
                tc_fence_after();
                issue_pv(t, 0, rv.slot, j == 0);
                if (!(ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_P_FULL + 2 * t + 1, par, 224 + t)))) break;
                tc_fence_after();
                issue_pv(t, 1, rv.slot, j == 0);
                if (t == ntq - 1 && leader) tc_commit(c.bars + (BAR_KV_EMPTY + rv.slot) * 8);
                if (more) {
                    if (t == 0 && !(ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_KV_FULL + rk.slot, rk.phase, 230)))) break;
                    tc_fence_after();
                    issue_qk(t, rk.slot);
                    if (t == ntq - 1 && leader) {
                        tc_commit(c.bars + (BAR_KV_EMPTY + rk.slot) * 8);
                        /* That was the last read of this item's Q tiles. */
                        if (j + 2 == nkv) tc_commit(c.bars + BAR_Q_EMPTY * 8);
                    }
                }
            }
        }
        for (int t = 0; t < ntq; t++) seen[t] += (uint32_t)nkv;
    }
    if (!ok) {
        /* Let what was issued finish before the tensor memory goes away. */
        if (leader) tc_commit(c.bars + BAR_DRAIN * 8);
        uint32_t bar = c.bars + BAR_DRAIN * 8;
        unsigned long long t0 = global_ns();
        while (!mbar_try_wait(bar, 0) && global_ns() - t0 < c.wait_ns) {}
    }
}

/* Valid-key bits of key tile j holding `nkeys` keys (bit b of word w = key
 * 32 w + b of the tile). */
__device__ __forceinline__ void tile_bits(const Params &p, int j, int nkeys, uint32_t bits[4]) {
#pragma unroll
    for (int w = 0; w < 4; w++) {
        int left = nkeys - 32 * w;
        uint32_t b = left >= 32 ? 0xFFFFFFFFu : (left <= 0 ? 0u : ((1u << left) - 1u));
        if (p.mask_bits) b &= p.mask_bits[j * 4 + w];    /* padded to whole tiles by the packer */
        bits[w] = b;
    }
}

/* Scores of masked / out-of-range keys become -inf. */
__device__ __forceinline__ void mask_chunk(uint32_t *v, uint32_t bits) {
#pragma unroll
    for (int i = 0; i < 32; i++)
        if (!((bits >> i) & 1u)) v[i] = 0xFF800000u;
}

/* Half an S row (64 scores) -> P (bf16 pairs into 32 columns at tP) and the
 * four partial row sums: one fp32 exponential per score. */
__device__ __forceinline__ void exp_half(const uint32_t *s, float sl2, float neg_ref, float *sum4, uint32_t tP) {
#pragma unroll
    for (int ch = 0; ch < 2; ch++) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            float x0 = fmaf(__uint_as_float(s[ch * 32 + 2 * i]), sl2, neg_ref);
            float x1 = fmaf(__uint_as_float(s[ch * 32 + 2 * i + 1]), sl2, neg_ref);
            float p0 = ex2(x0);
            float p1 = ex2(x1);
            sum4[(2 * i) & 3] += p0;
            sum4[(2 * i + 1) & 3] += p1;
            pk[i] = cvt_bf16x2(p0, p1);
        }
        tmem_st16(tP + ch * 16, pk);
    }
}

/* fp32 rows of a warp through its staging area. A thread owns one row of
 * the accumulator; memory wants eight threads per 128 contiguous bytes of a
 * row. Both helpers move 32 columns (128 bytes) of the warp's 32 rows, of
 * which the first `nvalid` exist; `base` points at row 0, rows are `ld`
 * floats apart. The staging rows are 128 bytes with their 16-byte chunks
 * XOR-swizzled by the row, free of bank conflicts on either side. */
__device__ __forceinline__ void rows_load_f32(uint32_t *dst, const float *base, size_t ld, int nvalid,
                                              unsigned char *stage_w, int lane) {
    const int ch = lane & 7;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int r = k * 4 + (lane >> 3);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < nvalid) v = __ldcg(reinterpret_cast<const uint4 *>(base + (size_t)r * ld + ch * 4));
        *reinterpret_cast<uint4 *>(stage_w + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    }
    __syncwarp();
#pragma unroll
    for (int c8 = 0; c8 < 8; c8++) {
        const uint4 v = *reinterpret_cast<const uint4 *>(stage_w + lane * 128 + ((c8 ^ (lane & 7)) << 4));
        dst[4 * c8] = v.x; dst[4 * c8 + 1] = v.y; dst[4 * c8 + 2] = v.z; dst[4 * c8 + 3] = v.w;
    }
    __syncwarp();
}
__device__ __forceinline__ void rows_store_f32(const uint32_t *src, float *base, size_t ld, int nvalid,
                                               unsigned char *stage_w, int lane) {
#pragma unroll
    for (int c8 = 0; c8 < 8; c8++)
        *reinterpret_cast<uint4 *>(stage_w + lane * 128 + ((c8 ^ (lane & 7)) << 4)) =
            make_uint4(src[4 * c8], src[4 * c8 + 1], src[4 * c8 + 2], src[4 * c8 + 3]);
    __syncwarp();
    const int ch = lane & 7;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int r = k * 4 + (lane >> 3);
        const uint4 v = *reinterpret_cast<const uint4 *>(stage_w + r * 128 + ((ch ^ (r & 7)) << 4));
        if (r < nvalid) __stcg(reinterpret_cast<uint4 *>(base + (size_t)r * ld + ch * 4), v);
    }
    __syncwarp();
}

/* One work item of query tile t. `cnt`: key tiles this tile has been through
 * before (the barrier phases run on over the items). False when aborting. */
__device__ __forceinline__ bool softmax_item(const Ctx &c, const Params &p, unsigned char *stage, uint32_t tmem, int t,
                                             int item, const Item &w, uint32_t cnt) {
    const int head = w.head, q0 = w.q0, nkv = w.nj;
    const int row = threadIdx.x & 127;                     /* row of the tile == TMEM lane */
    const uint32_t lane_base = (uint32_t)(row & ~31) << 16;
    const uint32_t tS = tmem + lane_base + t * 128;
    const uint32_t tO = tmem + lane_base + 256 + t * 128;
    const int qrow = q0 + t * kTileQ + row;
    const float sl2 = p.scale_log2;
    float m_ref = -INFINITY;     /* reference of the exponentials, in scaled log2 units */
    float l = 0.0f;
    bool ok = true;
    int si = source_of(p, w.j0);
    int src_last = (si + 1 < p.nsrc ? p.src[si + 1].tile0 : p.nkv) - 1;     /* last tile of the current source */

    for (int j = 0; j < nkv; j++) {
        /* One decision per warp: the TMEM accesses below are warp-collective. */
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_S_FULL + t, (cnt + j) & 1u, 300 + t)))) break;
        tc_fence_after();

        /* Only the last tile of a source can hold fewer than 128 keys. */
        const int jg = w.j0 + j;
        if (jg > src_last) {
            si++;
            src_last = (si + 1 < p.nsrc ? p.src[si + 1].tile0 : p.nkv) - 1;
        }
        int nkeys = kTileK;
        if (jg == src_last) nkeys = tile_keys(p.src[si], jg);
        IRIS_CHECK(c.status, si < p.nsrc && jg >= p.src[si].tile0 && jg <= src_last && nkeys >= 1 && nkeys <= kTileK, 921, jg);
        const bool partial = nkeys < kTileK || p.mask_bits != nullptr;
        uint32_t bits[4] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
        if (partial) tile_bits(p, jg, nkeys, bits);

        /* The whole S row of this thread: four loads in flight, one wait. */
        uint32_t s[128];
#pragma unroll
        for (int ch = 0; ch < 4; ch++) tmem_ld32(tS + ch * 32, s + ch * 32);
        tc_wait_ld();
        if (partial) {
#pragma unroll
            for (int ch = 0; ch < 4; ch++) mask_chunk(s + ch * 32, bits[ch]);
        }
        /* Row maximum over eight independent chains. */
        float mx8[8];
#pragma unroll
        for (int a = 0; a < 8; a++) mx8[a] = fmaxf(__uint_as_float(s[2 * a]), __uint_as_float(s[2 * a + 1]));
#pragma unroll
        for (int i = 16; i < 128; i += 16) {
#pragma unroll
            for (int a = 0; a < 8; a++)
                mx8[a] = max3(mx8[a], __uint_as_float(s[i + 2 * a]), __uint_as_float(s[i + 2 * a + 1]));
        }
        float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], fmaxf(mx8[5], fmaxf(mx8[6], mx8[7]))));
        float m_cand = fmaxf(m_ref, mx * sl2);

        if (j == 0) {
            m_ref = m_cand;
        } else {
            bool need = m_cand > m_ref + kRescaleThreshold;
            if (__any_sync(0xffffffffu, need)) {
                /* PV(j-1) of this tile has completed (it was issued before
                 * the QK that filled S) and PV(j) waits for our arrival: O
                 * is ours to rescale. */
                float alpha = need ? ex2(m_ref - m_cand) : 1.0f;
                if (need) {
                    l *= alpha;
                    m_ref = m_cand;
                }
#pragma unroll 1
                for (int i = 0; i < 4; i++) {
                    uint32_t o[32];
                    tmem_ld32(tO + i * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; e++) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                    tmem_st32(tO + i * 32, o);
                }
            }
        }

        /* P = 2^(s * scale_log2 - m_ref) as bf16 pairs over the first 64
         * columns of S (the row is in registers, so nothing is lost). A
         * masked (-inf) score gives an exact 0. */
        const float neg_ref = m_ref == -INFINITY ? 0.0f : -m_ref;
        float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            exp_half(s + 64 * h, sl2, neg_ref, sum4, tS + 32 * h);
            /* Hand each half of P to the MMA issuer as soon as it is stored. */
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(c.bars + (BAR_P_FULL + 2 * t + h) * 8);
        }
        l += (sum4[0] + sum4[2]) + (sum4[1] + sum4[3]);
    }

    /* Epilogue: O / l -> bf16 rows of the output slice of this head. */
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(c, BAR_O_DONE + t, (cnt + nkv - 1) & 1u, 310 + t));
    if (!ok) return false;
    tc_fence_after();
    const int lane = threadIdx.x & 31, wrow0 = row & ~31;

    /* Key split: each warp settles with its counterparts of the other parts
     * through a ticket. All but the last to arrive leave their unnormalised
     * rows, maxima and sums in the scratch of the query block and move on;
     * the last, which only ever waits for warps that are already writing,
     * folds them into its own and goes on to the output as if it had seen
     * every key. */
    float a_own = 1.0f;
    int nmerge = 0;
    const float *part_rows = nullptr;         /* the warp's 32 rows of the first partial */
    const float2 *part_ml_row = nullptr;      /* this row's (m, l) of the first partial */
    unsigned char *stage_w = stage + (size_t)(t * 4 + (wrow0 >> 5)) * 4096;
    if (p.nparts > 1) {
        const int others = p.nparts - 1;
        unsigned int *tk = p.tickets + ((size_t)w.qitem * 8 + t * 4 + (wrow0 >> 5)) * 2;
        float *prows = p.part_o + (((size_t)w.qitem * others) * 256 + t * kTileQ + wrow0) * kHeadDim;
        float2 *pml = p.part_ml + ((size_t)w.qitem * others) * 256 + t * kTileQ + row;
        unsigned int order = 0;
        if (lane == 0) order = atomicAdd(tk, 1u);
        order = __shfl_sync(0xffffffffu, order, 0);
        IRIS_CHECK(c.status, order < (unsigned)p.nparts && w.qitem < p.ticket_cap &&
                   (size_t)w.qitem * others + others <= (size_t)p.part_cap, 920, order);
        if (order < (unsigned)others) {
            float *mine = prows + (size_t)order * 256 * kHeadDim;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t o[64];
                tmem_ld32(tO + half * 64, o);
                tmem_ld32(tO + half * 64 + 32, o + 32);
                tc_wait_ld();
                rows_store_f32(o, mine + half * 64, kHeadDim, 32, stage_w, lane);
                rows_store_f32(o + 32, mine + half * 64 + 32, kHeadDim, 32, stage_w, lane);
            }
            __stcg(pml + (size_t)order * 256, make_float2(m_ref, l));
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(tk + 1, 1u);
            tc_fence_before();
            return true;
        }
        unsigned int ready = 1;
        if (lane == 0) {
            ready = word_wait(c, tk + 1, (uint32_t)others, 320 + t, (unsigned)item) ? 1u : 0u;
            tk[0] = 0u;                      /* the next launch finds the pair of words cleared */
            tk[1] = 0u;
        }
        ready = __shfl_sync(0xffffffffu, ready, 0);
        if (!ready) return false;
        __threadfence();
        float m_new = m_ref, l_new;
        for (int i = 0; i < others; i++) m_new = fmaxf(m_new, __ldcg(pml + (size_t)i * 256).x);
        a_own = m_ref == -INFINITY ? 0.0f : ex2(m_ref - m_new);
        l_new = a_own * l;
        for (int i = 0; i < others; i++) {
            const float2 ml = __ldcg(pml + (size_t)i * 256);
            l_new += ml.x == -INFINITY ? 0.0f : ex2(ml.x - m_new) * ml.y;
        }
        l = l_new;
        m_ref = m_new;
        nmerge = others;
        part_rows = prows;
        part_ml_row = pml;
    }
    const bool valid = qrow < p.seq_q;
    float inv = l > 0.0f ? 1.0f / l : 0.0f;

    /* Chunked state: this launch saw only part of the keys. lse = m + log2(l). */
    float w_prev = 0.0f, w_cur = 1.0f;
    if (p.acc_mode != 0 && valid) {
        float *lse_p = p.lse_acc + (size_t)head * p.seq_q + qrow;
        float lse_cur = l > 0.0f ? m_ref + log2f(l) : -INFINITY;
        if (p.acc_mode >= 2) {
            float lse_prev = *lse_p;
            float lse_new = fmaxf(lse_prev, lse_cur);
            if (lse_new == -INFINITY) {
                w_prev = 0.0f; w_cur = 0.0f;
            } else {
                float a = exp2f(lse_prev - lse_new), b = exp2f(lse_cur - lse_new);
                lse_new += log2f(a + b);
                w_prev = a / (a + b);
                w_cur = b / (a + b);
            }
            lse_cur = lse_new;
        }
        if (p.acc_mode != 3) *lse_p = lse_cur;
    }
    const bool write_state = p.acc_mode == 1 || p.acc_mode == 2;
    const bool read_state = p.acc_mode >= 2;
    const bool write_out = p.acc_mode == 0 || p.acc_mode == 3;
    const bool vec16 = (p.ldo & 7) == 0;
    uint16_t *orow = p.out ? p.out + (size_t)qrow * p.ldo + (size_t)head * kHeadDim : nullptr;

    /* Two passes of 64 columns. The bf16 rows go through a 4 KB staging area
     * private to the warp (32 rows x 128 bytes, 16-byte chunks XOR-swizzled by
     * the row so that neither side has bank conflicts): a thread owns a row
     * of the accumulator, but eight threads writing 128 contiguous bytes of
     * one output row is what the memory system wants. */
    const float f_all = inv * w_cur, f_cur = f_all * a_own;
    const int grow0 = q0 + t * kTileQ + wrow0;                       /* first row of this warp */
    const int nvalid = p.seq_q - grow0 < 32 ? (p.seq_q - grow0 < 0 ? 0 : p.seq_q - grow0) : 32;
    const size_t ld_acc = (size_t)p.heads * kHeadDim;
    float *acc_rows = p.acc_mode != 0 ? p.o_acc + (size_t)grow0 * ld_acc + (size_t)head * kHeadDim : nullptr;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        uint32_t o[64];
        tmem_ld32(tO + half * 64, o);
        tmem_ld32(tO + half * 64 + 32, o + 32);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 64; e++) o[e] = __float_as_uint(__uint_as_float(o[e]) * f_cur);
#pragma unroll 1
        for (int i = 0; i < nmerge; i++) {
            const float2 ml = __ldcg(part_ml_row + (size_t)i * 256);
            const float f_i = ml.x == -INFINITY ? 0.0f : f_all * ex2(ml.x - m_ref);
            const float *rows_i = part_rows + (size_t)i * 256 * kHeadDim;
#pragma unroll
            for (int sub = 0; sub < 2; sub++) {
                uint32_t pr[32];
                rows_load_f32(pr, rows_i + half * 64 + sub * 32, kHeadDim, 32, stage_w, lane);
#pragma unroll
                for (int e = 0; e < 32; e++)
                    o[sub * 32 + e] = __float_as_uint(fmaf(__uint_as_float(pr[e]), f_i, __uint_as_float(o[sub * 32 + e])));
            }
        }
        if (read_state) {
#pragma unroll
            for (int sub = 0; sub < 2; sub++) {
                uint32_t pr[32];
                rows_load_f32(pr, acc_rows + half * 64 + sub * 32, ld_acc, nvalid, stage_w, lane);
#pragma unroll
                for (int e = 0; e < 32; e++)
                    o[sub * 32 + e] = __float_as_uint(fmaf(__uint_as_float(pr[e]), w_prev, __uint_as_float(o[sub * 32 + e])));
            }
        }
        if (write_state) {
            rows_store_f32(o, acc_rows + half * 64, ld_acc, nvalid, stage_w, lane);
            rows_store_f32(o + 32, acc_rows + half * 64 + 32, ld_acc, nvalid, stage_w, lane);
        }
        if (write_out) {
            uint32_t pkd[32];
#pragma unroll
            for (int e = 0; e < 32; e++) pkd[e] = cvt_bf16x2(__uint_as_float(o[2 * e]), __uint_as_float(o[2 * e + 1]));
            if (vec16) {
#pragma unroll
                for (int ch = 0; ch < 8; ch++)
                    *reinterpret_cast<uint4 *>(stage_w + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
                        make_uint4(pkd[4 * ch], pkd[4 * ch + 1], pkd[4 * ch + 2], pkd[4 * ch + 3]);
                __syncwarp();
                const int ch = lane & 7;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const int r = k * 4 + (lane >> 3);
                    const uint4 val = *reinterpret_cast<const uint4 *>(stage_w + r * 128 + ((ch ^ (r & 7)) << 4));
                    const int grow = q0 + t * kTileQ + wrow0 + r;
                    if (grow < p.seq_q)
                        *reinterpret_cast<uint4 *>(p.out + (size_t)grow * p.ldo + (size_t)head * kHeadDim + half * 64 + ch * 8) = val;
                }
                __syncwarp();
            } else if (valid) {
#pragma unroll
                for (int e = 0; e < 32; e++) *reinterpret_cast<uint32_t *>(orow + half * 64 + e * 2) = pkd[e];
            }
        }
    }
    /* The reads of O above are complete (each was waited for); the fence
     * orders them before the arrival that lets the next item's PV start. */
    tc_fence_before();
    return true;
}

/* The softmax warpgroup of query tile t, over the work items of this CTA. */
__device__ __forceinline__ void softmax_wg(const Ctx &c, const Params &p, unsigned char *stage, uint32_t tmem, int t,
                                           const int *mail) {
    uint32_t cnt = 0;
    for (int n = 0;; n++) {
        const int item = sched_get(c, mail, n, 340 + t);
        if (item < 0) return;
        const Item w = item_of(p, item);
        if (t >= w.ntq) continue;
        if (!softmax_item(c, p, stage, tmem, t, item, w, cnt)) return;
        cnt += (uint32_t)w.nj;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
k_attention_sm100(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk0,
                  const __grid_constant__ CUtensorMap tmv0, const __grid_constant__ CUtensorMap tmk1,
                  const __grid_constant__ CUtensorMap tmv1, const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    /* The swizzled operand tiles need 1024-byte alignment. */
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_raw + (smem - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    Ctx c;
    c.bars = smem + kSmemBar;
    c.abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + kSmemAbort);
    c.status = p.status;
    c.wait_ns = p.wait_ns;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + kSmemTmemPtr);
    int *mail = reinterpret_cast<int *>(smem_gen + kSmemBar + kSmemSched);

    if (threadIdx.x == 0) {
        mbar_init(c.bars + BAR_Q_FULL * 8, 1);
        for (int s = 0; s < kStages; s++) {
            mbar_init(c.bars + (BAR_KV_FULL + s) * 8, 1);
            mbar_init(c.bars + (BAR_KV_EMPTY + s) * 8, 1);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(c.bars + (BAR_S_FULL + t) * 8, 1);
            mbar_init(c.bars + (BAR_P_FULL + 2 * t) * 8, 128);
            mbar_init(c.bars + (BAR_P_FULL + 2 * t + 1) * 8, 128);
            mbar_init(c.bars + (BAR_O_DONE + t) * 8, 1);
            mbar_init(c.bars + (BAR_SCHED_FULL + t) * 8, 1);
            mbar_init(c.bars + (BAR_SCHED_EMPTY + t) * 8, kSchedConsumers);
        }
        mbar_init(c.bars + BAR_Q_EMPTY * 8, 1);
        mbar_init(c.bars + BAR_DRAIN * 8, 1);
        *c.abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 9) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem + kSmemBar + kSmemTmemPtr), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    /* Launched with programmatic stream serialisation: everything above ran
     * while the kernel before this one (the prologue, an earlier key chunk)
     * was still finishing; nothing below may start before its memory is final. */
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp < 8) {
        /* The third warpgroup hands most of its registers to the softmax ones. */
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        softmax_wg(c, p, smem_gen + kSmemStage, tmem, warp >> 2, mail);
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (warp == 8 && lane == 0) {
            Maps m;
            m.q = &tmq;
            m.k[0] = &tmk0; m.v[0] = &tmv0;
            m.k[1] = &tmk1; m.v[1] = &tmv1;
            producer(c, p, m, smem, mail);
        }
        if (warp == 9) mma_issuer(c, p, smem, tmem, mail);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    /* The last CTA through leaves the work-list counters at zero for the
     * next launch (no CTA fetches after it has counted itself out). */
    if (threadIdx.x == 0 && p.sched) {
        __threadfence();
        if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
            p.sched[0] = 0u;
            p.sched[1] = 0u;
        }
    }
}

/* key_mask (int per key, 0 = ignore) -> one bit per key, padded with zero
 * bits to a whole number of 128-key tiles. */
__global__ void k_pack_mask(uint32_t *bits, const int *key_mask, int seq_k, int nwords) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= nwords) return;
    uint32_t b = 0;
    for (int i = 0; i < 32; i++) {
        int key = w * 32 + i;
        if (key < seq_k && key_mask[key] != 0) b |= 1u << i;
    }
    bits[w] = b;
}

/* Rows of a bf16 [seq, heads*128] slice set to zero (attention over no keys). */
__global__ void k_zero_rows(uint16_t *out, int ldo, int seq, int width) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t n = (size_t)seq * width;
    if (i < n) out[(i / width) * ldo + (i % width)] = 0;
}

}  // namespace sm100

/* ---------------- host side ---------------- */

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn(void) {
    static EncodeTiledFn fn = NULL;
    static int tried = 0;
    if (!tried) {
        tried = 1;
        void *sym = NULL;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
        else
            (void)cudaGetLastError();
    }
    return fn;
}

/* 2-D map over a bf16 [seq, width] column slice with row stride ld: box of
 * 64 columns x box_rows rows, 128-byte swizzle, zero fill outside. The
 * callers pass the same views block after block, so encoded maps are kept in
 * a small table keyed by the view (the map holds no data, only the address
 * and shape; a table entry stays valid for any buffer at that address). */
struct MapKey {
    const void *base;
    int seq, width, ld, box_rows;
};
static struct {
    MapKey key;
    CUtensorMap map;
    unsigned long long used;
} g_maps[64];
static unsigned long long g_map_clock = 0;

bool make_tensor_map(void *map_out, const void *base, int seq, int width, int ld, int box_rows) {
    CUtensorMap *map = static_cast<CUtensorMap *>(map_out);
    int victim = 0;
    for (int i = 0; i < 64; i++) {
        if (g_maps[i].used && g_maps[i].key.base == base && g_maps[i].key.seq == seq &&
            g_maps[i].key.width == width && g_maps[i].key.ld == ld && g_maps[i].key.box_rows == box_rows) {
            g_maps[i].used = ++g_map_clock;
            *map = g_maps[i].map;
            return true;
        }
        if (g_maps[i].used < g_maps[victim].used) victim = i;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error(IRIS_B200_ECUDA, "cuTensorMapEncodeTiled lookup", NULL);
        return false;
    }
    cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)seq};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof(msg), "CUresult %d", (int)r);
        set_error(IRIS_B200_ECUDA, "cuTensorMapEncodeTiled", msg);
        return false;
    }
    g_maps[victim].key = MapKey{base, seq, width, ld, box_rows};
    g_maps[victim].map = *map;
    g_maps[victim].used = ++g_map_clock;
    return true;
}

bool sm100_supported(const void *out, int ldo, const void *q, const void *k, const void *v, int ldi,
                     int heads, int kv_heads, int head_dim, int causal, float scale) {
    uintptr_t bits = (uintptr_t)out | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v;
    return head_dim == sm100::kHeadDim && heads == kv_heads && !causal && scale > 0.0f &&
           ldi % 8 == 0 && ldo % 2 == 0 && (bits & 15) == 0 && (ldo % 8 == 0 || ((uintptr_t)out & 3) == 0);
}

/* Library-owned device memory a launch needs besides its operands: the
 * work-list counters, the scratch of the key split and the packed key mask.
 * One set per stream that launches (launches on one stream run one after the
 * other; those of different streams may overlap, so they must not share).
 * Sets are recycled least recently used; before a set changes hands the
 * device is brought to rest. */
struct StreamScratch {
    cudaStream_t stream;
    int in_use;
    unsigned long long used;
    unsigned int *sched;           /* [16] words, two in use */
    size_t part_blocks;            /* 256-row partials the split scratch has room for */
    float *o;
    float2 *ml;
    size_t ticket_blocks;          /* query blocks the ticket array has room for */
    unsigned int *tickets;
    uint32_t *mask_bits;
    size_t mask_words;
};
static const int kScratchSets = 8;
static StreamScratch g_scratch[kScratchSets];
static unsigned long long g_scratch_clock = 0;

static void dev_free(void *p) {
    if (p) cuda_ok(cudaFree(p), "free");
}

static void scratch_free(StreamScratch *sc) {
    dev_free(sc->sched);
    dev_free(sc->o);
    dev_free(sc->ml);
    dev_free(sc->tickets);
    dev_free(sc->mask_bits);
    memset(sc, 0, sizeof(*sc));
}

/* NULL when nothing can be allocated: the launch then runs with the static
 * work list, without key split, and refuses key masks. */
static StreamScratch *scratch_of(cudaStream_t stream) {
    StreamScratch *sc = NULL, *lru = &g_scratch[0];
    for (int i = 0; i < kScratchSets; i++) {
        if (g_scratch[i].in_use && g_scratch[i].stream == stream) sc = &g_scratch[i];
        if (!g_scratch[i].in_use) {
            if (lru->in_use) lru = &g_scratch[i];
        } else if (lru->in_use && g_scratch[i].used < lru->used) {
            lru = &g_scratch[i];
        }
    }
    if (!sc) {
        sc = lru;
        if (sc->in_use) {
            /* Its last launches may still be running on a stream this code
             * knows nothing about any more. */
            cuda_ok(cudaDeviceSynchronize(), "sync");
            scratch_free(sc);
        }
        if (cudaMalloc((void **)&sc->sched, 64) != cudaSuccess || cudaMemset(sc->sched, 0, 64) != cudaSuccess) {
            (void)cudaGetLastError();
            scratch_free(sc);
            return NULL;
        }
        sc->in_use = 1;
        sc->stream = stream;
    }
    sc->used = ++g_scratch_clock;
    return sc;
}

/* Room for the partials and tickets of `nq` query blocks cut in `nparts`. */
static bool scratch_parts(StreamScratch *sc, size_t nq, int nparts) {
    const size_t blocks = nq * (size_t)(nparts - 1);
    if (blocks > sc->part_blocks || nq > sc->ticket_blocks) {
        cuda_ok(cudaStreamSynchronize(sc->stream), "sync");
        dev_free(sc->o);
        dev_free(sc->ml);
        dev_free(sc->tickets);
        sc->o = NULL;
        sc->ml = NULL;
        sc->tickets = NULL;
        sc->part_blocks = sc->ticket_blocks = 0;
        const size_t cap = blocks < 64 ? 64 : blocks, tcap = nq < 64 ? 64 : nq;
        if (cudaMalloc((void **)&sc->o, cap * 256 * sm100::kHeadDim * sizeof(float)) != cudaSuccess ||
            cudaMalloc((void **)&sc->ml, cap * 256 * sizeof(float2)) != cudaSuccess ||
            cudaMalloc((void **)&sc->tickets, tcap * 16 * sizeof(unsigned int)) != cudaSuccess ||
            cudaMemset(sc->tickets, 0, tcap * 16 * sizeof(unsigned int)) != cudaSuccess) {
            (void)cudaGetLastError();
            dev_free(sc->o);
            dev_free(sc->ml);
            dev_free(sc->tickets);
            sc->o = NULL;
            sc->ml = NULL;
            sc->tickets = NULL;
            return false;
        }
        sc->part_blocks = cap;
        sc->ticket_blocks = tcap;
    }
    return true;
}

static bool scratch_mask(StreamScratch *sc, size_t words) {
    if (words <= sc->mask_words) return true;
    cuda_ok(cudaStreamSynchronize(sc->stream), "sync");
    dev_free(sc->mask_bits);
    sc->mask_bits = NULL;
    sc->mask_words = 0;
    const size_t cap = words < 1024 ? 1024 : words * 2;
    if (cudaMalloc((void **)&sc->mask_bits, cap * 4) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    sc->mask_words = cap;
    return true;
}

static unsigned long long g_wait_ns = 1000000000ull;    /* 1 s */
static int g_inject_ticket = 0;                         /* host-side fault injection, one shot */
static int g_configured = 0, g_sm_count = 0;

void sm100_set_wait_limit_ns(unsigned long long ns) { g_wait_ns = ns ? ns : 1000000000ull; }
unsigned long long wait_limit_ns(void) { return g_wait_ns; }
void sm100_inject_stale_ticket(void) { g_inject_ticket = 1; }

/* Number of key parts that shortens the schedule most, by a model in units
 * of one key-tile iteration: the CTAs run ceil(items / CTAs) rounds of items
 * that each cost their tiles plus a fixed part (pipeline fill, output or
 * partial traffic, and the merge when there are parts). */
static int choose_parts(int nq, int nkv, int sms, int max_parts) {
    int best = 1;
    double best_cost = 0.0;
    for (int n = 1; n <= max_parts && n <= sm100::kMaxParts && (n == 1 || n <= nkv / 3); n++) {
        const long long items = (long long)nq * n;
        const long long ctas = items < sms ? items : sms;
        const double rounds = (double)((items + ctas - 1) / ctas);
        const double cost = rounds * ((double)nkv / n + 1.5 + (n > 1 ? 1.0 : 0.0));
        if (n == 1 || cost < best_cost * 0.97) {
            best = n;
            best_cost = cost;
        }
    }
    return best;
}

/* Pure host arithmetic of a launch: the first key tile of every run, the
 * number of key tiles, and how the keys of a query block are cut into parts
 * (the caller's boundaries, given as key rows and moved down to a tile
 * boundary, or equal numbers of tiles chosen by the cost model; can_split
 * false: one part). Returns IRIS_B200_OK or IRIS_B200_EINVAL. */
int plan_key_parts(const AttnArgs &a, int sm_count, bool can_split, KeyPlan *plan) {
    using namespace sm100;
    if (a.nsrc <= 0 || a.nsrc > kMaxSources || a.seq_q < 0 || a.heads <= 0) return IRIS_B200_EINVAL;
    int nkv = 0;
    for (int s = 0; s < a.nsrc; s++) {
        if (a.src[s].rows <= 0) return IRIS_B200_EINVAL;
        plan->tile0[s] = nkv;
        nkv += (a.src[s].rows + kTileK - 1) / kTileK;
    }
    plan->nkv = nkv;
    const int nq = ((a.seq_q + 2 * kTileQ - 1) / (2 * kTileQ)) * a.heads;
    int nparts = 1;
    if (can_split && a.nparts > 1)
        nparts = a.nparts > kMaxParts ? kMaxParts : a.nparts;
    else if (can_split && a.max_parts > 1)
        nparts = choose_parts(nq, nkv, sm_count, a.max_parts);
    plan->nparts = nparts;
    for (int i = 0; i <= nparts; i++) {
        if (a.nparts > 1 && nparts > 1 && i < nparts) {
            long long row = a.part_row[i], before = 0;
            int tile = nkv;
            for (int sidx = 0; sidx < a.nsrc; sidx++) {
                if (row < before + a.src[sidx].rows) {
                    tile = plan->tile0[sidx] + (int)((row - before) / kTileK);
                    break;
                }
                before += a.src[sidx].rows;
            }
            plan->part_tile[i] = tile;
        } else {
            plan->part_tile[i] = (int)((long long)nkv * i / nparts);
        }
    }
    plan->part_tile[0] = 0;
    for (int i = 0; i < nparts; i++)
        if (plan->part_tile[i + 1] <= plan->part_tile[i]) return IRIS_B200_EINVAL;
    return IRIS_B200_OK;
}

AttnArgs attn_args(uint16_t *out, int ldo, const uint16_t *q, int ldq, const uint16_t *k, const uint16_t *v,
                   int ldkv, int seq_q, int seq_k, int heads, float scale, const int *key_mask) {
    AttnArgs a = {};
    a.out = out;
    a.ldo = ldo;
    a.q = q;
    a.ldq = ldq;
    a.seq_q = seq_q;
    a.heads = heads;
    a.scale = scale;
    a.k[0] = k;
    a.v[0] = v;
    a.ldkv[0] = ldkv;
    a.nsrc = seq_k > 0 ? 1 : 0;
    a.src[0].view = 0;
    a.src[0].row0 = 0;
    a.src[0].rows = seq_k;
    a.src[0].arrive = -1;
    a.src[0].rows_per_word = 1;
    a.key_mask = key_mask;
    a.max_parts = AttnArgs::kMaxParts;
    return a;
}

int launch_attention_sm100(const AttnArgs &a) {
    using namespace sm100;
    if (!g_configured) {
        if (!cuda_ok(cudaFuncSetAttribute(k_attention_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                     "attention smem opt-in"))
            return IRIS_B200_ECUDA;
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sm_count <= 0) {
            (void)cudaGetLastError();
            g_sm_count = 148;
        }
        g_configured = 1;
    }
    const int heads = a.heads, seq_q = a.seq_q;
    if (a.nsrc <= 0) {
        if (a.acc_mode == 0) {
            size_t n = (size_t)seq_q * heads * kHeadDim;
            k_zero_rows<<<(unsigned)((n + 255) / 256), 256, 0, g.stream>>>(a.out, a.ldo, seq_q, heads * kHeadDim);
            return after_launch("attention (zero)") ? IRIS_B200_OK : IRIS_B200_ECUDA;
        }
        set_error(IRIS_B200_EINVAL, "attention", "empty key chunk");
        return IRIS_B200_EINVAL;
    }
    Params p = {};
    /* Sources -> tiles. */
    if (a.nsrc > kMaxSources || (a.key_mask && a.nsrc != 1)) {
        set_error(IRIS_B200_EINVAL, "attention", "too many key runs, or a key mask over more than one run");
        return IRIS_B200_EINVAL;
    }
    int view_rows[2] = {0, 0};
    int nkv = 0;
    for (int s = 0; s < a.nsrc; s++) {
        const AttnArgs::Source &in = a.src[s];
        if (in.rows <= 0 || in.row0 < 0 || in.view < 0 || in.view > 1 || !a.k[in.view] || !a.v[in.view] ||
            (in.arrive >= 0 && (!a.arrive || in.rows_per_word <= 0 ||
                                in.arrive + (in.rows - 1) / in.rows_per_word >= 32))) {
            set_error(IRIS_B200_EINVAL, "attention", "bad key run");
            return IRIS_B200_EINVAL;
        }
        KeySource &ks = p.src[s];
        ks.tile0 = nkv;
        ks.row0 = in.row0;
        ks.rows = in.rows;
        ks.view = in.view;
        ks.arrive = in.arrive;
        ks.rows_per_word = in.arrive >= 0 ? in.rows_per_word : 1;
        nkv += (in.rows + kTileK - 1) / kTileK;
        if (in.row0 + in.rows > view_rows[in.view]) view_rows[in.view] = in.row0 + in.rows;
    }
    p.nsrc = a.nsrc;
    p.nkv = nkv;
    p.view_rows[0] = view_rows[0];
    p.view_rows[1] = view_rows[1];
    p.arrive = a.arrive;
    p.arrive_seq = a.arrive_seq;

    StreamScratch *sc = a.no_scratch ? NULL : scratch_of(g.stream);
    if (a.key_mask) {
        const size_t words = (size_t)nkv * 4;
        if (!sc || !scratch_mask(sc, words)) {
            set_error(IRIS_B200_ENOMEM, "mask scratch", NULL);
            return IRIS_B200_ENOMEM;
        }
        k_pack_mask<<<(unsigned)((words + 127) / 128), 128, 0, g.stream>>>(sc->mask_bits, a.key_mask, a.src[0].rows,
                                                                           (int)words);
        if (!after_launch("attention (mask pack)")) return IRIS_B200_ECUDA;
        p.mask_bits = sc->mask_bits;
    }
    CUtensorMap tmq, tmk[2] = {}, tmv[2] = {};
    const int width = heads * kHeadDim;
    if (!make_tensor_map(&tmq, a.q, seq_q, width, a.ldq, kTileQ)) return IRIS_B200_ECUDA;
    for (int vw = 0; vw < 2; vw++) {
        if (view_rows[vw] == 0) {
            tmk[vw] = tmk[0];           /* never dereferenced */
            tmv[vw] = tmv[0];
        } else if (!make_tensor_map(&tmk[vw], a.k[vw], view_rows[vw], width, a.ldkv[vw], kTileK) ||
                   !make_tensor_map(&tmv[vw], a.v[vw], view_rows[vw], width, a.ldkv[vw], kTileK)) {
            return IRIS_B200_ECUDA;
        }
    }
    p.out = a.out;
    p.ldo = a.ldo;
    p.seq_q = seq_q;
    p.heads = heads;
    p.nqblk = (seq_q + 2 * kTileQ - 1) / (2 * kTileQ);
    p.nq = p.nqblk * heads;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = g.dev_status;
    p.wait_ns = g_wait_ns;
    p.o_acc = a.o_acc;
    p.lse_acc = a.lse_acc;
    p.acc_mode = a.acc_mode;
    p.sched = sc ? sc->sched : NULL;

    /* Key parts (none without scratch to merge through, or when the scratch cannot be had). */
    KeyPlan plan;
    if (plan_key_parts(a, g_sm_count, sc != NULL, &plan) != IRIS_B200_OK) {
        set_error(IRIS_B200_EINVAL, "attention", "empty key part");
        return IRIS_B200_EINVAL;
    }
    if (plan.nparts > 1 && !scratch_parts(sc, (size_t)p.nq, plan.nparts)) {
        plan_key_parts(a, g_sm_count, false, &plan);
    }
    const int nparts = plan.nparts;
    p.nparts = nparts;
    for (int i = 0; i <= nparts; i++) p.part_tile[i] = plan.part_tile[i];
    if (nparts > 1) {
        p.part_o = sc->o;
        p.part_ml = sc->ml;
        p.tickets = sc->tickets;
        p.part_cap = (int)sc->part_blocks;
        p.ticket_cap = (int)sc->ticket_blocks;
        if (g_inject_ticket) {
            /* Fault injection (tests): an arrival nobody made. Every part of
             * query block 0 then believes it is the last and waits for
             * partials that never come, until the wait limit ends the launch. */
            g_inject_ticket = 0;
            cuda_ok(cudaMemsetAsync(sc->tickets, 1, 1, g.stream), "ticket injection");
        }
    }
    p.items = p.nq * nparts;
    /* One CTA per SM at most (shared and tensor memory allow no more). */
    unsigned grid = (unsigned)(p.items < g_sm_count ? p.items : g_sm_count);
    /* Programmatic stream serialisation: the CTAs may be scheduled, and set
     * up their barriers and tensor memory, as soon as the kernel ahead on the
     * stream lets go of SMs; they wait for its completion inside the kernel. */
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, k_attention_sm100, tmq, tmk[0], tmv[0], tmk[1], tmv[1], p);
    g.launches++;
    return cuda_ok(err, "attention (tcgen05)") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

/* After a launch gave up on a wait: tickets and work-list counters may be
 * left half used. */
void sm100_reset_split(void) {
    cuda_ok(cudaDeviceSynchronize(), "sync");
    for (int i = 0; i < kScratchSets; i++) {
        StreamScratch *sc = &g_scratch[i];
        if (!sc->in_use) continue;
        if (sc->tickets) cuda_ok(cudaMemset(sc->tickets, 0, sc->ticket_blocks * 16 * sizeof(unsigned int)), "ticket clear");
        if (sc->sched) cuda_ok(cudaMemset(sc->sched, 0, 64), "work list clear");
    }
}

void sm100_release(void) {
    for (int i = 0; i < kScratchSets; i++)
        if (g_scratch[i].in_use) scratch_free(&g_scratch[i]);
    memset(g_maps, 0, sizeof(g_maps));
    gemm_release();
    g_configured = 0;              /* the next device needs its own opt-in */
    g_sm_count = 0;
}

}  // namespace iris_b200
