/* Internal launch functions shared between translation units. */
#pragma once
#include <stdint.h>

namespace iris_b200 {

int launch_attention_generic(uint16_t *out, int ldo, const uint16_t *q, const uint16_t *k,
                             const uint16_t *v, int ldi, int seq_q, int seq_k, int heads,
                             int kv_heads, int head_dim, float scale, int causal,
                             const int *key_mask);

bool sm100_supported(const void *out, int ldo, const void *q, const void *k, const void *v, int ldi,
                     int heads, int kv_heads, int head_dim, int causal, float scale);

/* One launch of the tcgen05 attention kernel. The keys are a sequence of
 * runs of rows taken from up to two K/V buffers ("views"); a run may be
 * guarded by arrival words that the kernel waits for before it loads the
 * run's rows. */
struct AttnArgs {
    enum { kMaxSources = 16, kMaxParts = 8 };
    uint16_t *out;
    int ldo;
    const uint16_t *q;
    int ldq, seq_q, heads;
    float scale;
    const uint16_t *k[2], *v[2];        /* view 0 / 1 */
    int ldkv[2];
    int nsrc;
    struct Source {
        int view, row0, rows;
        int arrive;                     /* first arrival word of the run, -1: none */
        int rows_per_word;              /* rows per arrival word */
    } src[kMaxSources];
    const uint32_t *arrive;             /* device words; arrived when (int)(word - arrive_seq) >= 0 */
    uint32_t arrive_seq;
    const int *key_mask;                /* single run only */
    int acc_mode;                       /* 0 plain; 1 / 2 / 3: first / middle / last chunk of a carried state */
    float *o_acc, *lse_acc;
    int max_parts;                      /* 1: never split the keys of a query block */
    int nparts;                         /* > 1: exactly these parts; part i starts at key row part_row[i],
                                           counted over the runs in order (moved down to a tile boundary) */
    long long part_row[kMaxParts + 1];
    bool no_scratch;                    /* use no library scratch: static work list, no key split, no mask */
};

/* How a launch cuts its keys (plan_key_parts): pure host arithmetic. */
struct KeyPlan {
    int nkv;                                   /* 128-key tiles over all runs */
    int tile0[AttnArgs::kMaxSources];          /* first tile of every run */
    int nparts;
    int part_tile[AttnArgs::kMaxParts + 1];    /* part i = tiles [part_tile[i], part_tile[i + 1]) */
};
int plan_key_parts(const AttnArgs &a, int sm_count, bool can_split, KeyPlan *plan);

/* Arguments of the plain case: one run of seq_k rows, split chosen by the library. */
AttnArgs attn_args(uint16_t *out, int ldo, const uint16_t *q, int ldq, const uint16_t *k, const uint16_t *v,
                   int ldkv, int seq_q, int seq_k, int heads, float scale, const int *key_mask);

int launch_attention_sm100(const AttnArgs &a);

/* Encodes (or finds in a small table) the TMA descriptor of a bf16 [rows, width]
 * matrix with row stride ld: boxes of 64 columns x box_rows rows, 128-byte
 * swizzle, zero fill outside. map_out: a CUtensorMap. */
bool make_tensor_map(void *map_out, const void *base, int rows, int width, int ld, int box_rows);

void sm100_release(void);

/* Clears the tickets and work-list counters (after a device wait timed out). */
void sm100_reset_split(void);

/* Limit of every wait inside the kernels (0 restores the default of 1 s). */
void sm100_set_wait_limit_ns(unsigned long long ns);
unsigned long long wait_limit_ns(void);

/* Per-device launch configuration of the GEMM is redone after a cleanup. */
void gemm_release(void);

/* Row-parallel GEMM: the fp32 rows of x [rows, in] . W [out, in]^T (row strides
 * ldx, ldw) are scattered to the ranks that own them: rank q owns the rows
 * [row_first[q], row_first[q + 1]) and receives them in slab[q] ([its rows,
 * out] fp32, local or peer memory); when the launch is through, the word
 * arrive[q] on every owner is set to seq. done: a zeroed device word. */
struct ScatterArgs {
    int nranks;
    const int *row_first;
    float *const *slab;
    uint32_t *const *arrive;
    uint32_t seq;
    unsigned int *done;
};
int launch_linear_scatter(const uint16_t *x, int ldx, const uint16_t *W, int ldw, int rows, int in, int out,
                          const ScatterArgs &sc);
/* x [rows, dim] += gate * (sum of nranks slabs), after the arrival words reached seq. */
int launch_residual_from_slabs(float *x, const float *slabs, size_t slab_stride, int nranks, const float *gate, int rows,
                               int dim, const uint32_t *arrive, uint32_t seq);

/* fp32 destination of a linear layer: y [rows, out] with row stride ld,
 * stored, or (accumulate) y += gate[c] * result with gate NULL meaning 1. */
struct F32Out {
    float *y;
    int ld;
    const float *gate;
    int accumulate;
    /* nseg > 0: one gate per run of rows instead (rows below seg_end[i] and
     * not below seg_end[i - 1] take seg_gate[i]; NULL: 1). */
    int nseg;
    int seg_end[4];
    const float *seg_gate[4];
};
int launch_linear_residual_segments(float *x_rows, int ldx, const uint16_t *a, int lda, const uint16_t *W, int ldw,
                                    const int *seg_end, const float *const *seg_gate, int nseg, int rows, int in, int out);

/* Gated-linear-unit destination of a linear layer: the last 2 * cols rows of W
 * are `cols` gate rows then `cols` up rows; y [rows, cols] (bf16, row stride
 * ld) = silu(gate) * up. */
struct GluOut {
    uint16_t *y;
    int ld;
    int cols;
};

/* A second row group of a linear layer: rows [split, rows) use these weights. */
struct SecondGroup {
    int split;
    const uint16_t *W;
    const float *wq, *wk, *gate;
};

/* One linear layer over the two streams of a double block (rows [0, split)
 * text, [split, rows) image; W / wq / wk / gate indexed by stream). Exactly
 * one kind of output: y32 != NULL: y32 [rows, out] (fp32, row stride ldy) +=
 * gate * product; else qkv [rows, 3 * heads * 128] (row stride ldy) with the
 * Q/K prologue when heads > 0, and / or act [rows, mlp] (row stride lda) =
 * silu(gate rows) * up rows when act != NULL. */
struct TwoStreamLinear {
    const uint16_t *x;
    int ldx;
    const uint16_t *W[2];
    int ldw;
    int rows, split, in, out;
    float *y32;
    uint16_t *qkv;
    int ldy;
    uint16_t *act;
    int lda, mlp;
    int heads;
    const float *wq[2], *wk[2], *gate[2];
    const float *rope_cos, *rope_sin;
    float eps;
};
int launch_linear_two(const TwoStreamLinear &a);

/* Rows of a linear layer's input that arrive while the kernel runs: rows
 * [row_first[q], row_first[q + 1]) are final once words[q] has reached seq. */
struct RowGuard {
    const uint32_t *words;
    int n;
    const int *row_first;
    uint32_t seq;
};
/* iris_b200_linear_glu on such an input (x with row stride ldx). */
int launch_linear_glu_guarded(uint16_t *qkv, int ldq, uint16_t *act, int lda, const uint16_t *x, int ldx, const uint16_t *W,
                              int rows, int in, int heads, int mlp, const float *wq, const float *wk, const float *rope_cos,
                              const float *rope_sin, float eps, const RowGuard &guard);
/* LayerNorm with modulation of this rank's rows, written to the same rows of
 * every destination (local or peer memory); once all rows are out, word[q] of
 * every destination is set to seq. done: a zeroed device word. */
struct GatherOut {
    int n;
    uint16_t *dst[16];
    uint32_t *word[16];
    uint32_t seq;
    unsigned int *done;
};
int launch_layer_norm_mod_gather(const GatherOut &out, const float *x, const float *shift, const float *scale, int rows,
                                 int dim, float eps);

/* Host-side fault injection: the next launch that splits its keys finds a
 * ticket that nobody took. */
void sm100_inject_stale_ticket(void);

/* A device wait ran out: a ring that was in use cannot go on (multi_gpu.cu). */
void ring_mark_failed(void);

/* Shared argument checks of the device-pointer attention entry points. */
int check_attention_args(const char *op, const void *out, const void *q, const void *k, const void *v, int ldo,
                         int ldq, int ldkv, int seq_q, int seq_k, int heads, int kv_heads, int head_dim);

}  // namespace iris_b200
