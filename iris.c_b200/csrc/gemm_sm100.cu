/*
 * QKV projection with the attention prologue as its epilogue, for sm_100a.
 *
 * y[rows, out] = x[rows, in] . W[out, in]^T, bf16 operands, fp32 accumulation
 * in tensor memory, bf16 result: the reference's iris_dev_linear_bf16
 * (iris_cuda.cu:463-506, a cuBLAS call). In the transformer blocks that GEMM
 * is followed at once by two iris_dev_head_norm_rope passes over the Q and K
 * column blocks of its output (iris_transformer_flux.c:3795-3801, 3832-3837).
 * A head is 128 columns, exactly half an N tile here, so the epilogue can do
 * the per-head RMSNorm and the pair rotation on the accumulator row it already
 * holds and the prologue's read-modify-write of Q and K disappears.
 *
 * Arithmetic of a Q / K head in the epilogue mirrors the two-kernel sequence
 * of the reference: the accumulator is first rounded to bf16 (what the GEMM
 * would have stored), then widened, normalised (inv = rsqrt(mean(x^2) + eps),
 * a = x * (inv * w)), rotated, and rounded once more (iris_cuda.cu:403-420).
 *
 * Tiles: 128 rows x 256 columns per CTA (MMA M = 128, N = 256, K = 16), K in
 * blocks of 64 through a four-stage TMA ring (48 KB per stage). Two fp32
 * accumulators of 256 columns fill the tensor memory, so the epilogue of a
 * tile runs under the main loop of the next. Persistent grid, tiles dealt
 * round-robin with the row tiles of one column tile next to each other (they
 * share W through L2).
 *
 * Warps (192 threads): 0 TMA producer, 1 MMA issuer and owner of the tensor
 * memory, 2-5 epilogue (thread = accumulator row; rows leave through a
 * swizzled staging area so that global memory sees whole 128-byte segments).
 * Waits are bounded like those of the attention kernel.
 */
#include <stdlib.h>

#include "common.cuh"

#include <cuda.h>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace iris_b200 {

namespace gemm {

using namespace sm100;

static constexpr int kTileM = 128, kTileN = 256, kBlockK = 64;
static constexpr int kStages = 4;
static constexpr int kBytesA = kTileM * kBlockK * 2;        /* 16 KB */
static constexpr int kBytesB = kTileN * kBlockK * 2;        /* 32 KB */
static constexpr int kStageBytes = kBytesA + kBytesB;
static constexpr int kThreads = 192;
static constexpr int kSmemStage = kStages * kStageBytes;    /* epilogue staging: 4 warps x 4 KB */
static constexpr int kSmemW = kSmemStage + 4 * 4096;        /* norm weights: wq[128] | wk[128] fp32, per row group */
static constexpr int kSmemBar = kSmemW + 2048;
static constexpr int kSmemBytes = kSmemBar + 256 + 1024;    /* + barriers + alignment slack */
static constexpr uint32_t kIdesc = idesc_bf16(kTileM, kTileN);

enum {
    BAR_FULL = 0,                       /* kStages */
    BAR_EMPTY = BAR_FULL + kStages,     /* kStages */
    BAR_ACC_FULL = BAR_EMPTY + kStages, /* 2 */
    BAR_ACC_EMPTY = BAR_ACC_FULL + 2,   /* 2 */
    BAR_DRAIN = BAR_ACC_EMPTY + 2,
    BAR_COUNT
};
static constexpr int kSmemTmemPtr = BAR_COUNT * 8;
static constexpr int kSmemAbort = kSmemTmemPtr + 4;
static constexpr int kMaxScatterRanks = 16;
static constexpr int kMaxSegments = 4;

struct Params {
    uint16_t *y;
    int ldy;
    int rows, in, out;
    int tiles_m, tiles_n;
    int norm_cols;              /* columns [0, norm_cols) are Q heads, [norm_cols, 2 norm_cols) K heads; 0: plain GEMM */
    const float *wq, *wk;       /* [128] */
    const float *rope_cos, *rope_sin;   /* [rows, 64] */
    float eps;
    unsigned int *status;
    unsigned long long wait_ns;
    /* Row-parallel mode (the out-projection after head-parallel attention):
     * the fp32 tile rows are not stored to y but scattered to the rank that
     * owns each row, into this rank's slab of the owner's staging buffer,
     * with plain stores over NVLink; the last CTA out then advances this
     * rank's arrival word on every owner. */
    int scatter;                /* 0: bf16 result to y; 1: fp32 rows to their owners; 2: fp32 rows to y32 */
    /* fp32 mode (the reference's iris_dev_linear_f32, iris_cuda.cu:560-584,
     * and, with accumulate, that followed by iris_dev_residual, :339-343, in
     * one pass): y32[r, c] = acc, or y32[r, c] += gate[c] * acc (gate NULL: 1). */
    float *y32;
    int ld32;
    int accumulate;
    const float *gate;
    /* Gated-linear-unit columns (the MLP half of a block's input projection):
     * from column tile glu_tile0 on, a tile is 128 gate columns next to their
     * 128 up columns (W rows glu_col0 + 128 j and glu_col0 + glu_cols + 128 j,
     * two TMA boxes per stage), and the epilogue stores silu(gate) * up, both
     * rounded to bf16 first as the reference's GEMM stores them
     * (iris_dev_linear_bf16 then k_swiglu, iris_cuda.cu:300-307), to y2. The
     * columns before glu_col0 are ordinary tiles. glu_tile0 == tiles_n: off. */
    int glu_tile0, glu_col0, glu_cols;
    uint16_t *y2;
    int ldy2;
    /* Two row groups with their own weights in one launch (the text and
     * image streams of a double block, whose rows are adjacent in every
     * buffer): rows [0, split) use the first W map, norm weights and gate,
     * rows [split, rows) the second. Row tiles never straddle the boundary:
     * group 0 has tiles_m0 of them, the rows a partial tile reads beyond its
     * group are computed and not stored. split == rows: one group. */
    int split, tiles_m0;
    const float *wq1, *wk1, *gate1;
    int ctas;                   /* 1, or 2: a row tile is 256 rows worked on by a CTA pair (k_linear_pair_sm100) */
    /* Rows of x that arrive while the kernel runs (an all-gather whose senders
     * store straight into x: the tensor-parallel blocks): rows [guard_first[q],
     * guard_first[q + 1]) are final once the word guard[q] has reached
     * guard_seq. The producer waits (bounded) for the owners of a row tile
     * before its first load of the tile. guard == NULL: everything is there. */
    const uint32_t *guard;
    int guard_n;
    int guard_first[kMaxScatterRanks + 1];
    uint32_t guard_seq;
    /* Gates by runs of rows that share the weights (the segments of a FLUX.3
     * block: text, image, reference rows, each with its own modulation):
     * rows below seg_end[i] (and not below seg_end[i - 1]) take seg_gate[i].
     * nseg == 0: the row group's gate. */
    int nseg;
    int seg_end[kMaxSegments];
    const float *seg_gate[kMaxSegments];
    /* Order of the work list: column tiles are taken in bands of band_n; inside
     * a band the tiles of one row tile are adjacent. The CTAs of the grid work
     * on ~148 consecutive tiles at a time, i.e. on 148 / band_n row tiles x
     * band_n column tiles, whose operands (A: 128 x in, W: 256 x in per tile)
     * should fit L2 together. band_n == 1: all row tiles of a column tile are
     * adjacent (small x, the input projections); band_n == tiles_n: all column
     * tiles of a row tile are adjacent (large x and in, the output projections). */
    int band_n;
    int nranks;
    int row_first[kMaxScatterRanks + 1];    /* rank q owns the rows [row_first[q], row_first[q + 1]) */
    float *slab[kMaxScatterRanks];          /* where this rank's partial rows of owner q go ([rows of q, out] fp32) */
    uint32_t *arrive[kMaxScatterRanks];     /* this rank's arrival word on owner q */
    uint32_t seq;
    unsigned int *done;                     /* CTAs that are through; zero between launches */
};

/* Row tile tm of a launch: its first row, the end of its row group, the group. */
struct RowTile {
    int m0, row_end, grp;
};
__host__ __device__ __forceinline__ RowTile row_tile(const Params &p, int tm, int rank = 0) {
    const int span = kTileM * p.ctas;           /* rows of a row tile; CTA `rank` of a pair takes the second half */
    if (tm < p.tiles_m0) return {tm * span + rank * kTileM, p.split, 0};
    return {p.split + (tm - p.tiles_m0) * span + rank * kTileM, p.rows, 1};
}

/* Work item `tile` of the list: its row tile and its column tile. */
__host__ __device__ __forceinline__ void tile_of(const Params &p, int tile, int *tm, int *nt) {
    const int per_band = p.tiles_m * p.band_n;
    const int band = tile / per_band, rem = tile - band * per_band;
    const int left = p.tiles_n - band * p.band_n;
    const int width = left < p.band_n ? left : p.band_n;
    *tm = rem / width;
    *nt = band * p.band_n + rem - *tm * width;
}

struct Ctx {
    uint32_t bars;
    volatile uint32_t *abort_flag;
    unsigned int *status;
    unsigned long long wait_ns;
    uint32_t peer_abort;        /* shared::cluster address of the other CTA's abort flag; 0: no pair */
};

__device__ __forceinline__ bool wait(const Ctx &c, int idx, uint32_t parity, int site) {
    const uint32_t bar = c.bars + idx * 8;
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 63u) {
            if (*c.abort_flag) return false;
            if (global_ns() - t0 > c.wait_ns || spin > (1u << 26)) {
                *c.abort_flag = 1u;
                if (c.peer_abort) st_cluster_u32(c.peer_abort, 1u);
                if (atomicCAS(c.status, 0u, 1u) == 0u) {
                    c.status[1] = (unsigned)site;
                    c.status[2] = blockIdx.x;
                    c.status[3] = parity;
                }
                return false;
            }
        }
    }
}

/* The rows [m0, m0 + kTileM) of x: wait for the arrival words of their owners. `arrived` remembers the owners seen. */
__device__ __forceinline__ bool rows_arrived(const Ctx &c, const Params &p, int m0, uint32_t *arrived) {
    if (!p.guard) return true;
    const int m1 = m0 + kTileM < p.rows ? m0 + kTileM : p.rows;
    for (int q = 0; q < p.guard_n; q++) {
        if (p.guard_first[q + 1] <= m0 || p.guard_first[q] >= m1 || ((*arrived >> q) & 1u)) continue;
        const unsigned long long t0 = global_ns();
        for (uint32_t spin = 0;; spin++) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.guard + q) : "memory");
            if ((int32_t)(v - p.guard_seq) >= 0) break;
            if ((spin & 7u) == 7u) {
                if (*c.abort_flag) return false;
                if (global_ns() - t0 > c.wait_ns || spin > (1u << 26)) {
                    *c.abort_flag = 1u;
                    if (c.peer_abort) st_cluster_u32(c.peer_abort, 1u);
                    if (atomicCAS(c.status, 0u, 1u) == 0u) {
                        c.status[1] = 480u;
                        c.status[2] = blockIdx.x;
                        c.status[3] = (unsigned)q;
                    }
                    return false;
                }
                __nanosleep(100);
            }
        }
        *arrived |= 1u << q;
        /* written by another GPU's stores; the loads below go through the asynchronous proxy */
        asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    return true;
}

__device__ __forceinline__ void producer(const Ctx &c, const Params &p, const CUtensorMap *tmx, const CUtensorMap *tmw0,
                                         const CUtensorMap *tmw1, uint32_t smem) {
    const int nkb = (p.in + kBlockK - 1) / kBlockK;
    int issued = 0;
    uint32_t arrived = 0u;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.tiles_m * p.tiles_n; tile += gridDim.x) {
        int tm, nt;
        tile_of(p, tile, &tm, &nt);
        const RowTile rt = row_tile(p, tm);
        const int m0 = rt.m0;
        const CUtensorMap *tmw = rt.grp ? tmw1 : tmw0;
        const bool halves = p.glu_tile0 < p.tiles_n;           /* W comes in two boxes of 128 rows */
        int n0 = nt * kTileN, n1 = n0 + kTileN / 2;
        if (nt >= p.glu_tile0) {
            n0 = p.glu_col0 + (nt - p.glu_tile0) * (kTileN / 2);
            n1 = n0 + p.glu_cols;
        }
        if (!(ok = rows_arrived(c, p, m0, &arrived))) break;
        for (int kb = 0; kb < nkb; kb++, issued++) {
            const int s = issued % kStages;
            if (issued >= kStages && !(ok = wait(c, BAR_EMPTY + s, ((issued / kStages) - 1) & 1u, 400 + s))) break;
            const uint32_t full = c.bars + (BAR_FULL + s) * 8;
            mbar_expect_tx(full, kStageBytes);
            tma_load_2d(smem + s * kStageBytes, tmx, kb * kBlockK, m0, full);
            tma_load_2d(smem + s * kStageBytes + kBytesA, tmw, kb * kBlockK, n0, full);
            if (halves) tma_load_2d(smem + s * kStageBytes + kBytesA + kBytesB / 2, tmw, kb * kBlockK, n1, full);
        }
    }
    if (*c.abort_flag) {
        /* Nobody may be consuming any more: wait for the copies still in flight. */
        for (int it = issued > kStages ? issued - kStages : 0; it < issued; it++)
            wait(c, BAR_FULL + it % kStages, (it / kStages) & 1u, 490);
    }
}

__device__ __forceinline__ void mma_issuer(const Ctx &c, const Params &p, uint32_t smem, uint32_t tmem) {
    const int nkb = (p.in + kBlockK - 1) / kBlockK;
    const uint32_t hi = (uint32_t)(make_desc(0, 0, 1024 / 16) >> 32);      /* 8 rows of 128 B */
    const uint32_t lo0 = (uint32_t)make_desc(smem, 1, 0);
    const bool leader = elect_one();
    int consumed = 0;
    bool ok = true;
    for (int tile = blockIdx.x, n = 0; ok && tile < p.tiles_m * p.tiles_n; tile += gridDim.x, n++) {
        const int buf = n & 1;
        /* The epilogue has emptied this accumulator (its use two tiles ago). */
        if (n >= 2 && !(ok = __all_sync(0xffffffffu, wait(c, BAR_ACC_EMPTY + buf, ((n >> 1) - 1) & 1u, 410 + buf)))) break;
        tc_fence_after();
        for (int kb = 0; kb < nkb; kb++, consumed++) {
            const int s = consumed % kStages;
            if (!(ok = __all_sync(0xffffffffu, wait(c, BAR_FULL + s, (consumed / kStages) & 1u, 420 + s)))) break;
            tc_fence_after();
            const uint32_t lo_a = lo0 + ((s * kStageBytes) >> 4), lo_b = lo_a + (kBytesA >> 4);
#pragma unroll
            for (int ks = 0; ks < kBlockK / 16; ks++) {
                if (leader)
                    mma_ss(tmem + buf * kTileN, ((uint64_t)hi << 32) | (lo_a + ks * 2), ((uint64_t)hi << 32) | (lo_b + ks * 2),
                           kIdesc, (kb | ks) != 0);
            }
            if (leader) tc_commit(c.bars + (BAR_EMPTY + s) * 8);
        }
        if (ok && leader) tc_commit(c.bars + (BAR_ACC_FULL + buf) * 8);
    }
    if (!ok) {
        if (leader) tc_commit(c.bars + BAR_DRAIN * 8);
        const uint32_t bar = c.bars + BAR_DRAIN * 8;
        const unsigned long long t0 = global_ns();
        while (!mbar_try_wait(bar, 0) && global_ns() - t0 < c.wait_ns) {}
    }
}

/* 32 rows x 64 bf16 columns (128 bytes per row) of one warp to global memory
 * through its staging area: thread `lane` holds its row's 32 packed words;
 * the 16-byte chunks are XOR-swizzled by the row so that neither the row-wise
 * writes nor the segment-wise reads conflict. Rows >= nrows and columns >=
 * ncols (a multiple of 8) are not stored. */
__device__ __forceinline__ void store_rows_bf16(const uint32_t *pk, uint16_t *base, size_t ld, int nrows, int ncols,
                                                unsigned char *stage_w, int lane) {
#pragma unroll
    for (int ch = 0; ch < 8; ch++)
        *reinterpret_cast<uint4 *>(stage_w + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
            make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
    __syncwarp();
    const int ch = lane & 7;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int r = k * 4 + (lane >> 3);
        const uint4 val = *reinterpret_cast<const uint4 *>(stage_w + r * 128 + ((ch ^ (r & 7)) << 4));
        if (r < nrows && ch * 8 < ncols) *reinterpret_cast<uint4 *>(base + (size_t)r * ld + ch * 8) = val;
    }
    __syncwarp();
}

/* 32 rows x 32 fp32 columns of one warp to the owners of the rows: staged like
 * the bf16 rows, each 128-byte row segment then goes to the slab of the rank
 * that owns the row (ncols a multiple of 4). */
__device__ __forceinline__ void scatter_rows_f32(const uint32_t *src, const Params &p, int wrow0, int nrows, int c0,
                                                 int ncols, unsigned char *stage_w, int lane) {
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
        if (r < nrows && ch * 4 < ncols) {
            const int row = wrow0 + r;
            int q = 0;
            while (q + 1 < p.nranks && row >= p.row_first[q + 1]) q++;
            float *dst = p.slab[q] + (size_t)(row - p.row_first[q]) * p.out + c0 + ch * 4;
            *reinterpret_cast<uint4 *>(dst) = v;
        }
    }
    __syncwarp();
}

/* fp32 destination of a tile (scatter == 2). Each warp owns 32 rows; it goes
 * through the tile in chunks of 32 columns: the accumulator chunk comes from
 * TMEM, is transposed through the swizzled staging area so that eight lanes
 * cover 128 contiguous bytes of a row, and is stored, or added in place with
 * a per-column gate. Every element belongs to exactly one warp of one tile,
 * so the read-modify-write needs no atomics. The old values of chunk c + 1
 * are fetched before chunk c is processed: a load issued next to the store it
 * feeds would leave every row segment waiting a full memory round trip. */
struct XChunk {
    float4 v[8];
};

__device__ __forceinline__ const float *gate_of_row(const Params &p, const float *group_gate, int row) {
    if (p.nseg == 0) return group_gate;
    int i = 0;
    while (i + 1 < p.nseg && row >= p.seg_end[i]) i++;
    return p.seg_gate[i];
}

__device__ __forceinline__ void load_old(XChunk &x, const Params &p, int wrow0, int nrows, int c0, int lane) {
    const int ch = lane & 7;
    const int ncols = p.out - c0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int r = k * 4 + (lane >> 3);
        x.v[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r < nrows && ch * 4 < ncols)
            x.v[k] = *reinterpret_cast<const float4 *>(p.y32 + (size_t)(wrow0 + r) * p.ld32 + c0 + ch * 4);
    }
}

__device__ __forceinline__ void tile_f32(const Params &p, const float *group_gate, uint32_t tmem_tile, int wrow0, int nrows,
                                         int col0, unsigned char *stage_w, int lane) {
    const int ch = lane & 7;
    XChunk cur, next;
    if (p.accumulate) load_old(next, p, wrow0, nrows, col0, lane);
#pragma unroll 1
    for (int c = 0; c < kTileN / 32; c++) {
        const int c0 = col0 + c * 32;
        if (c0 >= p.out) break;
        uint32_t acc[32];
        tmem_ld32(tmem_tile + c * 32, acc);
        cur = next;
        if (p.accumulate && c + 1 < kTileN / 32 && c0 + 32 < p.out) load_old(next, p, wrow0, nrows, c0 + 32, lane);
        tc_wait_ld();
#pragma unroll
        for (int c8 = 0; c8 < 8; c8++)
            *reinterpret_cast<uint4 *>(stage_w + lane * 128 + ((c8 ^ (lane & 7)) << 4)) =
                make_uint4(acc[4 * c8], acc[4 * c8 + 1], acc[4 * c8 + 2], acc[4 * c8 + 3]);
        __syncwarp();
        const bool col_ok = ch * 4 < p.out - c0;
        float4 g4 = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if (p.nseg == 0 && group_gate && col_ok) g4 = *reinterpret_cast<const float4 *>(group_gate + c0 + ch * 4);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int r = k * 4 + (lane >> 3);
            float4 v = *reinterpret_cast<const float4 *>(stage_w + r * 128 + ((ch ^ (r & 7)) << 4));
            if (r < nrows && col_ok) {
                if (p.nseg > 0) {
                    const float *gs = gate_of_row(p, group_gate, wrow0 + r);
                    g4 = gs ? *reinterpret_cast<const float4 *>(gs + c0 + ch * 4) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                }
                if (p.accumulate) {
                    const float4 x = cur.v[k];
                    v = make_float4(fmaf(g4.x, v.x, x.x), fmaf(g4.y, v.y, x.y), fmaf(g4.z, v.z, x.z), fmaf(g4.w, v.w, x.w));
                }
                *reinterpret_cast<float4 *>(p.y32 + (size_t)(wrow0 + r) * p.ld32 + c0 + ch * 4) = v;
            }
        }
        __syncwarp();
    }
}

/* Where an epilogue finds its tiles and barriers: CTA `rank` of a pair (0 for
 * a single CTA) takes the tiles first, first + stride, ...; acc_empty_remote
 * != 0: the barrier array of the pair's first CTA (shared::cluster address),
 * on which both CTAs' epilogue warps arrive. */
struct EpiSched {
    int first, stride, rank;
    int bar_acc_full, bar_acc_empty;
    uint32_t acc_empty_remote;
};

__device__ __forceinline__ void acc_release(const Ctx &c, const EpiSched &e, int buf) {
    if (e.acc_empty_remote) mbar_arrive_cluster(e.acc_empty_remote + (e.bar_acc_empty + buf) * 8);
    else mbar_arrive(c.bars + (e.bar_acc_empty + buf) * 8);
}

__device__ __forceinline__ void epilogue(const Ctx &c, const Params &p, unsigned char *stage, const float *w_smem,
                                         uint32_t tmem, const EpiSched &e) {
    const int lane = threadIdx.x & 31;
    const int quarter = (threadIdx.x >> 5) & 3;                 /* TMEM lane quarter of this warp */
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    unsigned char *stage_w = stage + quarter * 4096;
    for (int tile = e.first, n = 0; tile < p.tiles_m * p.tiles_n; tile += e.stride, n++) {
        const int buf = n & 1;
        int tm, nt;
        tile_of(p, tile, &tm, &nt);
        const RowTile rt = row_tile(p, tm, e.rank);
        const int m0 = rt.m0, n0 = nt * kTileN;     /* n0: ordinary tiles only */
        if (!__all_sync(0xffffffffu, wait(c, e.bar_acc_full + buf, (n >> 1) & 1u, 430 + buf))) return;
        tc_fence_after();
        const int row = m0 + row_in_tile;
        const int wrow0 = m0 + quarter * 32;
        const int nrows = rt.row_end - wrow0 < 32 ? (rt.row_end - wrow0 < 0 ? 0 : rt.row_end - wrow0) : 32;
        const bool row_ok = row < rt.row_end;
        if (p.scatter == 2) {
            tile_f32(p, rt.grp ? p.gate1 : p.gate, tmem + lane_base + buf * kTileN, wrow0, nrows, n0, stage_w, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) acc_release(c, e, buf);
            continue;
        }
        if (nt >= p.glu_tile0) {
            const int cbase = (nt - p.glu_tile0) * (kTileN / 2);            /* column of y2 */
#pragma unroll 1
            for (int pass = 0; pass < 2; pass++) {
                uint32_t gt[64], up[64], pk[32];
                tmem_ld32(tmem + lane_base + buf * kTileN + pass * 64, gt);
                tmem_ld32(tmem + lane_base + buf * kTileN + pass * 64 + 32, gt + 32);
                tmem_ld32(tmem + lane_base + buf * kTileN + 128 + pass * 64, up);
                tmem_ld32(tmem + lane_base + buf * kTileN + 128 + pass * 64 + 32, up + 32);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    const uint32_t g2 = cvt_bf16x2(__uint_as_float(gt[2 * e]), __uint_as_float(gt[2 * e + 1]));
                    const uint32_t u2 = cvt_bf16x2(__uint_as_float(up[2 * e]), __uint_as_float(up[2 * e + 1]));
                    const float g0 = bf_lo(g2), g1 = bf_hi(g2);
                    pk[e] = cvt_bf16x2(__fdividef(g0, 1.0f + __expf(-g0)) * bf_lo(u2),
                                       __fdividef(g1, 1.0f + __expf(-g1)) * bf_hi(u2));
                }
                const int c0 = cbase + pass * 64;
                const int ncols = p.glu_cols - c0 < 64 ? (p.glu_cols - c0 < 0 ? 0 : p.glu_cols - c0) : 64;
                store_rows_bf16(pk, p.y2 + (size_t)wrow0 * p.ldy2 + c0, (size_t)p.ldy2, nrows, ncols, stage_w, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) acc_release(c, e, buf);
            continue;
        }
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            const int col0 = n0 + half * 128;
            if (col0 >= p.out) break;
            /* 0 / 1: a Q / K head (norm + rotation), 2: plain columns */
            const int kind = col0 < p.norm_cols ? 0 : (col0 < 2 * p.norm_cols ? 1 : 2);
            uint32_t acc[128];
#pragma unroll
            for (int ch = 0; ch < 4; ch++) tmem_ld32(tmem + lane_base + buf * kTileN + half * 128 + ch * 32, acc + ch * 32);
            tc_wait_ld();
            if (p.scatter) {
#pragma unroll
                for (int sub = 0; sub < 4; sub++) {
                    const int c0 = col0 + sub * 32;
                    const int ncols = p.out - c0 < 32 ? (p.out - c0 < 0 ? 0 : p.out - c0) : 32;
                    scatter_rows_f32(acc + sub * 32, p, wrow0, nrows, c0, ncols, stage_w, lane);
                }
                continue;
            }
            float inv = 1.0f;
            if (kind < 2) {
                /* What the GEMM would have stored, then the sum of squares of that. */
                float ss0 = 0.0f, ss1 = 0.0f;
#pragma unroll
                for (int e = 0; e < 128; e += 2) {
                    const uint32_t pkd = cvt_bf16x2(__uint_as_float(acc[e]), __uint_as_float(acc[e + 1]));
                    const float a = bf_lo(pkd), b = bf_hi(pkd);
                    acc[e] = __float_as_uint(a);
                    acc[e + 1] = __float_as_uint(b);
                    ss0 = fmaf(a, a, ss0);
                    ss1 = fmaf(b, b, ss1);
                }
                inv = rsqrtf((ss0 + ss1) * (1.0f / 128.0f) + p.eps);
            }
            const float *w = w_smem + rt.grp * 256 + (kind == 1 ? 128 : 0);
            const float4 *cosr = reinterpret_cast<const float4 *>(p.rope_cos + (size_t)(row_ok ? row : 0) * 64);
            const float4 *sinr = reinterpret_cast<const float4 *>(p.rope_sin + (size_t)(row_ok ? row : 0) * 64);
#pragma unroll
            for (int pass = 0; pass < 2; pass++) {              /* 64 columns = 32 pairs per pass */
                uint32_t pk[32];
                if (kind < 2) {
#pragma unroll
                    for (int q4 = 0; q4 < 8; q4++) {
                        const float4 cc = cosr[pass * 8 + q4], sn = sinr[pass * 8 + q4];
                        const float cj[4] = {cc.x, cc.y, cc.z, cc.w}, sj[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const int e = pass * 64 + q4 * 8 + 2 * j;
                            const float a = __uint_as_float(acc[e]) * (inv * w[e]);
                            const float b = __uint_as_float(acc[e + 1]) * (inv * w[e + 1]);
                            pk[q4 * 4 + j] = cvt_bf16x2(a * cj[j] - b * sj[j], b * cj[j] + a * sj[j]);
                        }
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e++)
                        pk[e] = cvt_bf16x2(__uint_as_float(acc[pass * 64 + 2 * e]), __uint_as_float(acc[pass * 64 + 2 * e + 1]));
                }
                const int c0 = col0 + pass * 64;
                const int ncols = p.out - c0 < 64 ? (p.out - c0 < 0 ? 0 : p.out - c0) : 64;
                store_rows_bf16(pk, p.y + (size_t)wrow0 * p.ldy + c0, (size_t)p.ldy, nrows, ncols, stage_w, lane);
            }
        }
        /* Every read of this accumulator has been waited for. */
        tc_fence_before();
        __syncwarp();
        if (lane == 0) acc_release(c, e, buf);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
k_linear_sm100(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw,
               const __grid_constant__ CUtensorMap tmw1, const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_raw + (smem - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    Ctx c;
    c.bars = smem + kSmemBar;
    c.abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + kSmemAbort);
    c.status = p.status;
    c.wait_ns = p.wait_ns;
    c.peer_abort = 0u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + kSmemTmemPtr);
    float *w_smem = reinterpret_cast<float *>(smem_gen + kSmemW);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(c.bars + (BAR_FULL + s) * 8, 1);
            mbar_init(c.bars + (BAR_EMPTY + s) * 8, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(c.bars + (BAR_ACC_FULL + b) * 8, 1);
            mbar_init(c.bars + (BAR_ACC_EMPTY + b) * 8, 4);          /* one arrival per epilogue warp */
        }
        mbar_init(c.bars + BAR_DRAIN * 8, 1);
        *c.abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem + kSmemBar + kSmemTmemPtr), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (p.norm_cols > 0)
        for (int i = threadIdx.x; i < 512; i += kThreads) {
            const float *src = i < 256 ? (i < 128 ? p.wq : p.wk) : (i < 384 ? p.wq1 : p.wk1);
            w_smem[i] = src[i & 127];
        }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) producer(c, p, &tmx, &tmw, &tmw1, smem);
    } else if (warp == 1) {
        mma_issuer(c, p, smem, tmem);
    } else {
        const EpiSched e = {(int)blockIdx.x, (int)gridDim.x, 0, BAR_ACC_FULL, BAR_ACC_EMPTY, 0u};
        epilogue(c, p, smem_gen + kSmemStage, w_smem, tmem, e);
    }

    if (p.scatter == 1) __threadfence_system();          /* this thread's rows are out before the CTA counts itself out */
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    /* Row-parallel mode: once every CTA's rows are on their way (each fenced
     * at system scope above), the last CTA tells every owner that this rank's
     * partial sums of the call have arrived. A launch that gave up tells nobody. */
    if (p.scatter == 1 && threadIdx.x == 0) {
        const bool aborted = *c.abort_flag != 0u;
        __threadfence();
        const unsigned int prev = atomicAdd(p.done, aborted ? 0x10000u + 1u : 1u);
        if ((prev & 0xFFFFu) == gridDim.x - 1) {
            const bool any_aborted = aborted || (prev >> 16) != 0u;
            *p.done = 0u;
            if (!any_aborted) {
                __threadfence_system();
                for (int q = 0; q < p.nranks; q++)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.arrive[q]), "r"(p.seq) : "memory");
            }
        }
    }
}

/* ------------------------------------------------------------------------
 * CTA pairs: the same GEMM with a 256 x 256 tile per pair of CTAs
 * (tcgen05.mma.cta_group::2). Each CTA holds 128 rows of x and HALF of the W
 * tile per stage (32 KB instead of 48 KB, so six stages fit), the pair's
 * first CTA issues the MMAs, which read both halves of W from the two CTAs'
 * shared memory and write 128 x 256 accumulators into each CTA's TMEM. Per
 * unit of work every SM moves a third less through its shared memory, which
 * is what bounds the single-CTA kernel. Loads are plain TMA loads (each CTA
 * fetches what it holds; nothing is multicast); their byte counts go to the
 * first CTA's FULL barrier. EMPTY and ACC_FULL barriers of both CTAs are
 * signalled by the MMA commits; both CTAs' epilogue warps arrive on the first
 * CTA's ACC_EMPTY barrier. Every wait is bounded as in the single-CTA kernel,
 * and a CTA that gives up raises the peer's abort flag too.
 * ------------------------------------------------------------------------ */
static constexpr int kPairStages = 6;
static constexpr int kPairBytesB = kBytesB / 2;
static constexpr int kPairStageBytes = kBytesA + kPairBytesB;      /* 32 KB per CTA */
static_assert(kPairStages * kPairStageBytes == kSmemStage, "the pair kernel reuses the single-CTA shared-memory layout");
static constexpr uint32_t kPairIdesc = idesc_bf16(2 * kTileM, kTileN);
enum {
    PBAR_FULL = 0,
    PBAR_EMPTY = PBAR_FULL + kPairStages,
    PBAR_ACC_FULL = PBAR_EMPTY + kPairStages,
    PBAR_ACC_EMPTY = PBAR_ACC_FULL + 2,
    PBAR_DRAIN = PBAR_ACC_EMPTY + 2,
    PBAR_COUNT
};
static constexpr int kPairTmemPtr = PBAR_COUNT * 8;
static constexpr int kPairAbort = kPairTmemPtr + 4;
static_assert(kPairAbort + 4 <= 256, "barrier area");

__device__ __forceinline__ void pair_producer(const Ctx &c, const Params &p, const CUtensorMap *tmx, const CUtensorMap *tmw0,
                                              const CUtensorMap *tmw1, uint32_t smem, int rank, int first, int stride) {
    const int nkb = (p.in + kBlockK - 1) / kBlockK;
    const uint32_t full0 = map_to_cta(c.bars + PBAR_FULL * 8, 0);          /* the first CTA's FULL barriers */
    int issued = 0;
    uint32_t arrived = 0u;
    bool ok = true;
    for (int tile = first; ok && tile < p.tiles_m * p.tiles_n; tile += stride) {
        int tm, nt;
        tile_of(p, tile, &tm, &nt);
        const RowTile rt = row_tile(p, tm, rank);
        const CUtensorMap *tmw = rt.grp ? tmw1 : tmw0;
        /* this CTA's 128 rows of W: an ordinary tile's first or second half, or the gate or the up rows */
        int n = nt * kTileN + rank * (kTileN / 2);
        if (nt >= p.glu_tile0) n = p.glu_col0 + (nt - p.glu_tile0) * (kTileN / 2) + rank * p.glu_cols;
        if (!(ok = rows_arrived(c, p, rt.m0, &arrived))) break;
        for (int kb = 0; kb < nkb; kb++, issued++) {
            const int s = issued % kPairStages;
            if (issued >= kPairStages && !(ok = wait(c, PBAR_EMPTY + s, ((issued / kPairStages) - 1) & 1u, 600 + s))) break;
            if (rank == 0) mbar_expect_tx(c.bars + (PBAR_FULL + s) * 8, 2 * kPairStageBytes);
            tma_load_2d_pair(smem + s * kPairStageBytes, tmx, kb * kBlockK, rt.m0, full0 + s * 8);
            tma_load_2d_pair(smem + s * kPairStageBytes + kBytesA, tmw, kb * kBlockK, n, full0 + s * 8);
        }
    }
    if (*c.abort_flag && rank == 0) {
        /* Nobody may be consuming any more: wait for the pair's copies still in flight. */
        for (int it = issued > kPairStages ? issued - kPairStages : 0; it < issued; it++)
            wait(c, PBAR_FULL + it % kPairStages, (it / kPairStages) & 1u, 690);
    }
}

__device__ __forceinline__ void pair_mma_issuer(const Ctx &c, const Params &p, uint32_t smem, uint32_t tmem, int first,
                                                int stride) {
    const int nkb = (p.in + kBlockK - 1) / kBlockK;
    const uint32_t hi = (uint32_t)(make_desc(0, 0, 1024 / 16) >> 32);      /* 8 rows of 128 B */
    const uint32_t lo0 = (uint32_t)make_desc(smem, 1, 0);
    const bool leader = elect_one();
    int consumed = 0;
    bool ok = true;
    for (int tile = first, n = 0; ok && tile < p.tiles_m * p.tiles_n; tile += stride, n++) {
        const int buf = n & 1;
        /* Both CTAs' epilogues have emptied this accumulator (its use two tiles ago). */
        if (n >= 2 && !(ok = __all_sync(0xffffffffu, wait(c, PBAR_ACC_EMPTY + buf, ((n >> 1) - 1) & 1u, 610 + buf)))) break;
        tc_fence_after();
        for (int kb = 0; kb < nkb; kb++, consumed++) {
            const int s = consumed % kPairStages;
            if (!(ok = __all_sync(0xffffffffu, wait(c, PBAR_FULL + s, (consumed / kPairStages) & 1u, 620 + s)))) break;
            tc_fence_after();
            const uint32_t lo_a = lo0 + ((s * kPairStageBytes) >> 4), lo_b = lo_a + (kBytesA >> 4);
#pragma unroll
            for (int ks = 0; ks < kBlockK / 16; ks++) {
                if (leader)
                    mma_ss_pair(tmem + buf * kTileN, ((uint64_t)hi << 32) | (lo_a + ks * 2),
                                ((uint64_t)hi << 32) | (lo_b + ks * 2), kPairIdesc, (kb | ks) != 0);
            }
            if (leader) tc_commit_pair(c.bars + (PBAR_EMPTY + s) * 8, 3);
        }
        if (ok && leader) tc_commit_pair(c.bars + (PBAR_ACC_FULL + buf) * 8, 3);
    }
    if (!ok) {
        if (leader) tc_commit_pair(c.bars + PBAR_DRAIN * 8, 1);
        const uint32_t bar = c.bars + PBAR_DRAIN * 8;
        const unsigned long long t0 = global_ns();
        while (!mbar_try_wait(bar, 0) && global_ns() - t0 < c.wait_ns) {}
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
k_linear_pair_sm100(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw,
                    const __grid_constant__ CUtensorMap tmw1, const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_raw + (smem - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_cta_rank();
    const int first = (int)(blockIdx.x >> 1), stride = (int)(gridDim.x >> 1);

    Ctx c;
    c.bars = smem + kSmemBar;
    c.abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + kPairAbort);
    c.status = p.status;
    c.wait_ns = p.wait_ns;
    c.peer_abort = map_to_cta(smem + kSmemBar + kPairAbort, (uint32_t)(rank ^ 1));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + kPairTmemPtr);
    float *w_smem = reinterpret_cast<float *>(smem_gen + kSmemW);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; s++) {
            mbar_init(c.bars + (PBAR_FULL + s) * 8, 1);
            mbar_init(c.bars + (PBAR_EMPTY + s) * 8, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(c.bars + (PBAR_ACC_FULL + b) * 8, 1);
            mbar_init(c.bars + (PBAR_ACC_EMPTY + b) * 8, 8);         /* four epilogue warps in each CTA */
        }
        mbar_init(c.bars + PBAR_DRAIN * 8, 1);
        *c.abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem + kSmemBar + kPairTmemPtr), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    if (p.norm_cols > 0)
        for (int i = threadIdx.x; i < 512; i += kThreads) {
            const float *src = i < 256 ? (i < 128 ? p.wq : p.wk) : (i < 384 ? p.wq1 : p.wk1);
            w_smem[i] = src[i & 127];
        }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();               /* the peer's barriers exist before anything arrives on them */
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) pair_producer(c, p, &tmx, &tmw, &tmw1, smem, rank, first, stride);
    } else if (warp == 1) {
        if (rank == 0) pair_mma_issuer(c, p, smem, tmem, first, stride);
    } else {
        const EpiSched e = {first, stride, rank, PBAR_ACC_FULL, PBAR_ACC_EMPTY, map_to_cta(c.bars, 0)};
        epilogue(c, p, smem_gen + kSmemStage, w_smem, tmem, e);
    }

    /* Neither CTA leaves, or frees its TMEM, while the other may still read its
     * shared memory or arrive on its barriers. */
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

/* Owner side of the row-parallel mode: x[r, c] += gate[c] * sum over the
 * ranks' slabs (gate NULL: plain sum), after every rank's arrival word has
 * reached the call's sequence number (bounded wait; a word that does not come
 * is reported in the status word and nothing is added). The reference does the
 * same arithmetic in iris_dev_residual (iris_cuda.cu:339-343) on one GPU. */
__global__ void k_residual_from_slabs(float *x, const float *slabs, size_t slab_stride, int nranks, const float *gate,
                                      int rows, int dim, const uint32_t *arrive, uint32_t seq, unsigned long long wait_ns,
                                      unsigned int *status) {
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
        int ok = 1;
        const unsigned long long t0 = global_ns();
        for (int r = 0; r < nranks && ok; r++) {
            for (uint32_t spin = 0;; spin++) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(arrive + r) : "memory");
                if ((int32_t)(v - seq) >= 0) break;
                if ((spin & 7u) == 7u) {
                    if (global_ns() - t0 > wait_ns || spin > (1u << 26)) {
                        if (atomicCAS(status, 0u, 1u) == 0u) {
                            status[1] = 500u;
                            status[2] = blockIdx.x;
                            status[3] = (unsigned)r;
                        }
                        ok = 0;
                        break;
                    }
                    __nanosleep(100);
                }
            }
        }
        ok_s = ok;
    }
    __syncthreads();
    if (!ok_s) return;
    const size_t n4 = (size_t)rows * dim / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < nranks; r++) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(slabs + (size_t)r * slab_stride) + i);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        const int c = (int)((i * 4) % (size_t)dim);
        float4 g4 = make_float4(1.f, 1.f, 1.f, 1.f);
        if (gate) g4 = *reinterpret_cast<const float4 *>(gate + c);
        float4 xv = reinterpret_cast<float4 *>(x)[i];
        xv.x += g4.x * sum.x; xv.y += g4.y * sum.y; xv.z += g4.z * sum.z; xv.w += g4.w * sum.w;
        reinterpret_cast<float4 *>(x)[i] = xv;
    }
}

}  // namespace gemm

/* The tile grid of a launch: row tiles per row group, column tiles (ordinary
 * ones, then the gate|up pairs), and the order of the work list. m-fastest
 * order keeps every row tile of x plus a few column tiles of W in flight;
 * when that does not fit L2 comfortably and all of W is smaller, the list goes
 * through the columns of a row tile first (all of W and 1/tiles_n of the
 * concurrently processed x in flight). */
static void plan_grid(gemm::Params *p, int rows, int split, int in, int out, int glu_cols, int sm_count, int ctas = 1) {
    using namespace gemm;
    p->rows = rows;
    p->in = in;
    p->out = out;
    p->split = split;
    p->ctas = ctas;
    const int span = kTileM * ctas;
    p->tiles_m0 = (split + span - 1) / span;
    p->tiles_m = p->tiles_m0 + (rows - split + span - 1) / span;
    p->tiles_n = (out + kTileN - 1) / kTileN;
    p->glu_tile0 = p->tiles_n;
    p->glu_col0 = out;
    p->glu_cols = glu_cols;
    p->tiles_n += (glu_cols + kTileN / 2 - 1) / (kTileN / 2);
    const double a_tile = (double)span * in * 2, w_tile = (double)kTileN * in * 2;
    const double m_fast = p->tiles_m * a_tile + ((double)sm_count / ctas / (p->tiles_m > 0 ? p->tiles_m : 1) + 1) * w_tile;
    p->band_n = 1;
    if (m_fast > 96e6 && p->tiles_n * w_tile < m_fast) p->band_n = p->tiles_n;
}

static int g_gemm_configured = 0;
static int g_pair_mode = 1;             /* CTA pairs unless iris_b200_linear_cta_pairs(0) */
static int g_pair_clusters = 0;         /* CTA pairs that can be resident at once */

void gemm_release(void) {
    g_gemm_configured = 0;
    g_pair_clusters = 0;
}

/* y [rows, out] (row stride ldy) = x [rows, in] . W [out, in]^T; with heads > 0
 * the first 2 * heads * 128 columns are Q and K heads that get the prologue. */
static int launch_linear(uint16_t *y, int ldy, const uint16_t *x, int ldx, const uint16_t *W, int ldw, int rows, int in,
                         int out, int heads, const float *wq, const float *wk, const float *rope_cos,
                         const float *rope_sin, float eps, const ScatterArgs *sc, const char *op,
                         const F32Out *f32 = NULL, const GluOut *glu = NULL, const SecondGroup *g2 = NULL,
                         const RowGuard *guard = NULL) {
    using namespace gemm;
    if (!require_device(op)) return IRIS_B200_ENODEV;
    if ((!y && !sc && !f32 && !(glu && out == 0)) || (f32 && (!f32->y || f32->ld < out || f32->ld % 4 != 0 || ((uintptr_t)f32->y & 15) != 0 ||
                                        ((uintptr_t)f32->gate & 15) != 0 || f32->nseg < 0 || f32->nseg > kMaxSegments ||
                                        sc || heads > 0)) ||
        !x || !W || rows < 0 || in <= 0 || out < 0 || (out == 0 && !glu) || (y && ldy < out) || heads < 0 || ldx < in || ldw < in ||
        (heads > 0 && (!wq || !wk || !rope_cos || !rope_sin || 2 * heads * 128 > out)) ||
        (sc && (sc->nranks < 1 || sc->nranks > kMaxScatterRanks))) {
        set_error(IRIS_B200_EINVAL, op, "bad argument");
        return IRIS_B200_EINVAL;
    }
    const uintptr_t bits = (uintptr_t)y | (uintptr_t)x | (uintptr_t)W | (uintptr_t)rope_cos | (uintptr_t)rope_sin;
    if ((bits & 15) != 0 || in % 8 != 0 || out % 8 != 0 || ldy % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) {
        set_error(IRIS_B200_EUNSUPPORTED, op, "operands must be 16-byte aligned, in / out / row strides multiples of 8");
        return IRIS_B200_EUNSUPPORTED;
    }
    /* With glu, `out` counts the ordinary columns only (may be 0); W has out + 2 * glu->cols rows. The ordinary
     * columns end on a half tile (an odd number of 128-column heads is fine): the other half of that last tile is
     * computed from the gate rows that follow and never stored. */
    if (glu && (!glu->y || glu->cols <= 0 || glu->cols % 8 != 0 || glu->ld < glu->cols || glu->ld % 8 != 0 ||
                ((uintptr_t)glu->y & 15) != 0 || out % (kTileN / 2) != 0 || sc || f32)) {
        set_error(IRIS_B200_EINVAL, op, "bad gated-linear-unit argument");
        return IRIS_B200_EINVAL;
    }
    if (g2 && (g2->split < 0 || g2->split > rows || !g2->W || ((uintptr_t)g2->W & 15) != 0 || ((uintptr_t)g2->gate & 15) != 0 ||
               (heads > 0 && (!g2->wq || !g2->wk)) || sc)) {
        set_error(IRIS_B200_EINVAL, op, "bad second row group");
        return IRIS_B200_EINVAL;
    }
    if (rows == 0) return IRIS_B200_OK;
    if (!g_gemm_configured) {
        if (!cuda_ok(cudaFuncSetAttribute(k_linear_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                     "linear smem opt-in"))
            return IRIS_B200_ECUDA;
        g_gemm_configured = 1;
    }
    /* CTA pairs for everything but the row-parallel scatter (whose completion count is per CTA) */
    int ctas = g_pair_mode && !sc ? 2 : 1;
    if (ctas == 2 && !g_pair_clusters) {
        if (!cuda_ok(cudaFuncSetAttribute(k_linear_pair_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                     "linear smem opt-in"))
            return IRIS_B200_ECUDA;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(g.sm_count & ~1));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, k_linear_pair_sm100, &cfg) != cudaSuccess || n < 1) {
            (void)cudaGetLastError();
            n = -1;                     /* pairs cannot be placed: stay with single CTAs */
        }
        g_pair_clusters = n;
    }
    if (ctas == 2 && g_pair_clusters < 1) ctas = 1;
    CUtensorMap tmx, tmw, tmw1;
    const int w_rows = glu ? out + 2 * glu->cols : out;
    const int w_box = glu || ctas == 2 ? kTileN / 2 : kTileN;
    if (!make_tensor_map(&tmx, x, rows, in, ldx, kTileM) || !make_tensor_map(&tmw, W, w_rows, in, ldw, w_box) ||
        !make_tensor_map(&tmw1, g2 ? g2->W : W, w_rows, in, ldw, w_box))
        return IRIS_B200_ECUDA;
    Params p = {};
    p.y = y;
    p.ldy = ldy;
    p.rows = rows;
    p.in = in;
    p.out = out;
    plan_grid(&p, rows, g2 ? g2->split : rows, in, out, glu ? glu->cols : 0, g.sm_count, ctas);
    p.wq1 = g2 ? g2->wq : wq;
    p.wk1 = g2 ? g2->wk : wk;
    p.gate1 = g2 ? g2->gate : (f32 ? f32->gate : NULL);
    if (glu) {
        p.y2 = glu->y;
        p.ldy2 = glu->ld;
    }
    p.norm_cols = heads * 128;
    p.wq = wq;
    p.wk = wk;
    p.rope_cos = rope_cos;
    p.rope_sin = rope_sin;
    p.eps = eps;
    p.status = g.dev_status;
    p.wait_ns = wait_limit_ns();
    if (sc) {
        p.scatter = 1;
        p.nranks = sc->nranks;
        for (int q = 0; q <= sc->nranks; q++) p.row_first[q] = sc->row_first[q];
        for (int q = 0; q < sc->nranks; q++) {
            p.slab[q] = sc->slab[q];
            p.arrive[q] = sc->arrive[q];
        }
        p.seq = sc->seq;
        p.done = sc->done;
    }
    if (guard) {
        if (guard->n < 1 || guard->n > kMaxScatterRanks || !guard->words || guard->row_first[guard->n] != rows) {
            set_error(IRIS_B200_EINVAL, op, "bad row guards");
            return IRIS_B200_EINVAL;
        }
        p.guard = guard->words;
        p.guard_n = guard->n;
        for (int q = 0; q <= guard->n; q++) p.guard_first[q] = guard->row_first[q];
        p.guard_seq = guard->seq;
    }
    if (f32) {
        p.scatter = 2;
        p.y32 = f32->y;
        p.ld32 = f32->ld;
        p.accumulate = f32->accumulate;
        p.gate = f32->gate;
        p.nseg = f32->nseg;
        for (int i = 0; i < f32->nseg; i++) {
            p.seg_end[i] = f32->seg_end[i];
            p.seg_gate[i] = f32->seg_gate[i];
        }
    }
#ifdef IRIS_B200_TUNE
    if (const char *e = getenv("IRIS_B200_BAND_N")) {
        const int v = atoi(e);
        if (v > 0) p.band_n = v < p.tiles_n ? v : p.tiles_n;
    }
#endif
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    if (ctas == 2) {
        const unsigned clusters = (unsigned)(tiles < g_pair_clusters ? tiles : g_pair_clusters);
        k_linear_pair_sm100<<<2 * clusters, kThreads, kSmemBytes, g.stream>>>(tmx, tmw, tmw1, p);
        return after_launch(op) ? IRIS_B200_OK : IRIS_B200_ECUDA;
    }
    const unsigned grid = (unsigned)(tiles < g.sm_count ? tiles : g.sm_count);
    k_linear_sm100<<<grid, kThreads, kSmemBytes, g.stream>>>(tmx, tmw, tmw1, p);
    return after_launch(op) ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

int launch_linear_scatter(const uint16_t *x, int ldx, const uint16_t *W, int ldw, int rows, int in, int out,
                          const ScatterArgs &sc) {
    return launch_linear(NULL, 0, x, ldx, W, ldw, rows, in, out, 0, NULL, NULL, NULL, NULL, 0.0f, &sc, "outproj");
}

int launch_residual_from_slabs(float *x, const float *slabs, size_t slab_stride, int nranks, const float *gate, int rows,
                               int dim, const uint32_t *arrive, uint32_t seq) {
    if (rows <= 0) return IRIS_B200_OK;
    const size_t n4 = (size_t)rows * dim / 4;
    size_t blocks = (n4 + 255) / 256;
    if (blocks > (size_t)g.sm_count * 8) blocks = (size_t)g.sm_count * 8;
    gemm::k_residual_from_slabs<<<(unsigned)blocks, 256, 0, g.stream>>>(x, slabs, slab_stride, nranks, gate, rows, dim, arrive,
                                                                        seq, wait_limit_ns(), g.dev_status);
    return after_launch("outproj residual") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

}  // namespace iris_b200

using namespace iris_b200;

extern "C" void iris_dev_linear_bf16(uint16_t *y, const uint16_t *x, const uint16_t *W, int rows, int in, int out) {
    launch_linear(y, out, x, in, W, in, rows, in, out, 0, NULL, NULL, NULL, NULL, 0.0f, NULL, "linear_bf16");
}

/* Same arithmetic as the reference's iris_dev_linear_f32 (iris_cuda.cu:560-584):
 * bf16 operands, fp32 accumulation, fp32 result. */
extern "C" void iris_dev_linear_f32(float *y, const uint16_t *x, const uint16_t *W, int rows, int in, int out) {
    F32Out f = {};
    f.y = y;
    f.ld = out;
    launch_linear(NULL, 0, x, in, W, in, rows, in, out, 0, NULL, NULL, NULL, NULL, 0.0f, NULL, "linear_f32", &f);
}

extern "C" int iris_b200_linear_residual(float *x_rows, int ldx, const uint16_t *a, int lda, const uint16_t *W, int ldw,
                                         const float *gate, int rows, int in, int out) {
    F32Out f = {};
    f.y = x_rows;
    f.ld = ldx;
    f.gate = gate;
    f.accumulate = 1;
    return launch_linear(NULL, 0, a, lda, W, ldw, rows, in, out, 0, NULL, NULL, NULL, NULL, 0.0f, NULL, "linear_residual",
                         &f);
}

/* iris_b200_linear_residual with one gate per run of rows (a gate may be NULL: 1). */
int iris_b200::launch_linear_residual_segments(float *x_rows, int ldx, const uint16_t *a, int lda, const uint16_t *W, int ldw,
                                               const int *seg_end, const float *const *seg_gate, int nseg, int rows, int in,
                                               int out) {
    F32Out f = {};
    f.y = x_rows;
    f.ld = ldx;
    f.accumulate = 1;
    if (nseg < 1 || nseg > gemm::kMaxSegments) {
        set_error(IRIS_B200_EINVAL, "linear_residual", "1 to 4 segments");
        return IRIS_B200_EINVAL;
    }
    f.nseg = nseg;
    for (int i = 0; i < nseg; i++) {
        f.seg_end[i] = seg_end[i];
        f.seg_gate[i] = seg_gate[i];
        if (((uintptr_t)seg_gate[i] & 15) != 0) {
            set_error(IRIS_B200_EUNSUPPORTED, "linear_residual", "gates must be 16-byte aligned");
            return IRIS_B200_EUNSUPPORTED;
        }
    }
    return launch_linear(NULL, 0, a, lda, W, ldw, rows, in, out, 0, NULL, NULL, NULL, NULL, 0.0f, NULL, "linear_residual", &f);
}

int iris_b200::launch_linear_glu_guarded(uint16_t *qkv, int ldq, uint16_t *act, int lda, const uint16_t *x, int ldx,
                                         const uint16_t *W, int rows, int in, int heads, int mlp, const float *wq,
                                         const float *wk, const float *rope_cos, const float *rope_sin, float eps,
                                         const RowGuard &guard) {
    const GluOut glu = {act, lda, mlp};
    return launch_linear(qkv, ldq, x, ldx, W, in, rows, in, 3 * heads * 128, heads, wq, wk, rope_cos, rope_sin, eps, NULL,
                         "linear_glu (gathered rows)", NULL, &glu, NULL, &guard);
}

extern "C" int iris_b200_linear_glu(uint16_t *qkv, int ldq, uint16_t *act, int lda, const uint16_t *x, const uint16_t *W,
                                    int rows, int in, int heads, int mlp, const float *wq, const float *wk,
                                    const float *rope_cos, const float *rope_sin, float eps) {
    const GluOut glu = {act, lda, mlp};
    return launch_linear(qkv, ldq, x, in, W, in, rows, in, 3 * heads * 128, heads, wq, wk, rope_cos, rope_sin, eps, NULL,
                         "linear_glu", NULL, &glu);
}

/* The two streams of a double block in one launch: rows [0, split) against
 * the first set of weights, rows [split, rows) against the second. */
int iris_b200::launch_linear_two(const TwoStreamLinear &a) {
    const SecondGroup g2 = {a.split, a.W[1], a.wq[1], a.wk[1], a.gate[1]};
    F32Out f = {};
    f.y = a.y32;
    f.ld = a.ldy;
    f.gate = a.gate[0];
    f.accumulate = 1;
    const GluOut glu = {a.act, a.lda, a.mlp};
    const int out = a.y32 ? a.out : 3 * a.heads * 128;
    return launch_linear(a.y32 ? NULL : a.qkv, a.y32 ? 0 : a.ldy, a.x, a.ldx, a.W[0], a.ldw, a.rows, a.in, out, a.heads, a.wq[0],
                         a.wk[0], a.rope_cos, a.rope_sin, a.eps, NULL, "linear (two streams)", a.y32 ? &f : NULL,
                         a.act ? &glu : NULL, &g2);
}

extern "C" int iris_b200_linear_cta_pairs(int enable) {
    const int was = g_pair_mode;
    if (enable >= 0) g_pair_mode = enable ? 1 : 0;
    return was;
}

extern "C" int iris_b200_linear_plan(int rows, int split, int in, int out, int glu_cols, int sm_count, int *tiles_m,
                                     int *tiles_n, int *band_n, int *order, int cap) {
    if (rows < 0 || split < 0 || split > rows || in <= 0 || out < 0 || glu_cols < 0 || sm_count <= 0 || !tiles_m || !tiles_n ||
        !band_n)
        return -1;
    gemm::Params p = {};
    plan_grid(&p, rows, split, in, out, glu_cols, sm_count);
    *tiles_m = p.tiles_m;
    *tiles_n = p.tiles_n;
    *band_n = p.band_n;
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    if (order) {
        for (long long t = 0; t < tiles && t < cap; t++) {
            int tm, nt;
            gemm::tile_of(p, (int)t, &tm, &nt);
            const gemm::RowTile rt = gemm::row_tile(p, tm);
            order[4 * t] = rt.m0;
            order[4 * t + 1] = rt.row_end;
            order[4 * t + 2] = nt;
            order[4 * t + 3] = nt >= p.glu_tile0;
        }
    }
    return tiles > 0x7fffffff ? -1 : (int)tiles;
}

extern "C" int iris_b200_linear_qk_norm_rope(uint16_t *y, int ldy, const uint16_t *x, const uint16_t *W,
                                             int rows, int in, int out, int heads,
                                             const float *wq, const float *wk,
                                             const float *rope_cos, const float *rope_sin, float eps) {
    return launch_linear(y, ldy, x, in, W, in, rows, in, out, heads, wq, wk, rope_cos, rope_sin, eps, NULL,
                         "linear_qk_norm_rope");
}
