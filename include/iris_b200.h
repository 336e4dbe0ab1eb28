/*
 * Additions of the B200 implementation to the reference's operator surface.
 *
 * Nothing here has a counterpart in the reference unless a comment says
 * which reference code it stands in for: the reference is single device,
 * single stream and reports errors only on stderr. These entry points add a
 * status word, stream sharing, device-side timing, a one-launch Q+K
 * prologue, kernel selection for tests, stream-ordered copies, attention over
 * key runs that arrive over time, and the multi-GPU decompositions of the
 * attention (head shards, CFG split, ring sequence parallelism).
 */
#ifndef IRIS_B200_H
#define IRIS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ----------------------------------------------------------- */

enum {
    IRIS_B200_OK = 0,
    IRIS_B200_EINVAL = 1,       /* argument outside the documented domain */
    IRIS_B200_ECUDA = 2,        /* a CUDA runtime / driver call failed */
    IRIS_B200_ETIMEOUT = 3,     /* a bounded wait inside a kernel ran out */
    IRIS_B200_ENODEV = 4,       /* iris_dev_init() has not succeeded */
    IRIS_B200_ENOMEM = 5,       /* device allocation failed */
    IRIS_B200_EUNSUPPORTED = 6, /* no kernel for this argument combination */
    IRIS_B200_ECOMM = 7,        /* collective transport failed, or the ring is unusable after a failure */
    IRIS_B200_EPROTO = 8,       /* ring ranks disagree (row counts, chunk sizes, sequence numbers) */
    IRIS_B200_ECHECK = 9        /* a device-side self-check of the -DIRIS_B200_CHECK build did not hold */
};

/* First error since the last clear (0 = none). The void operations of
 * iris_dev.h record their failures here as well as printing them, the
 * extension the reference lacks (iris_cuda.cu:108-111 only prints). */
int iris_b200_last_error(void);
void iris_b200_clear_error(void);
const char *iris_b200_strerror(int code);

/* Waits for the stream, then reads the device-side status word written by
 * kernels whose internal waits are bounded (mbarrier / flag waits give up
 * after a time limit instead of spinning forever). Returns the resulting
 * last error. */
int iris_b200_check_device_status(void);

/* Limit of every wait inside the kernels, in microseconds (0 restores the
 * default of one second). Applies to the launches that follow. A host that
 * knows how long a peer may legitimately take (ring steps) sets it to that;
 * tests set a few milliseconds to make a wait run out. */
int iris_b200_set_wait_limit_us(unsigned int us);

/* Host-side fault injection for tests of the failure paths (nothing faults or
 * hangs on the GPU: the affected launch gives up at the wait limit and reports
 * IRIS_B200_ETIMEOUT). STALE_TICKET: the next launch that splits its keys
 * finds an arrival ticket nobody took, so the parts of one query block wait
 * for a partial result that never comes. One shot. */
enum { IRIS_B200_FAULT_STALE_TICKET = 1 };
int iris_b200_inject_fault(int what);

/* ---- device and stream ------------------------------------------------- */

/* Device ordinal used by the next iris_dev_init() (default 0, the
 * reference's fixed choice, iris_cuda.cu:122). One process per GPU. */
int iris_b200_set_device(int ordinal);

/* Run all operations on a stream owned by the caller (a cudaStream_t cast
 * to void *) instead of the internal one. Call after iris_dev_init(). This
 * is how the two hot operations are embedded next to another backend that
 * owns the stream. NULL restores the internal stream. */
int iris_b200_attach_stream(void *cuda_stream);
/* The same switch without the wait for the work already enqueued: for hosts
 * that run independent calls side by side on several streams (the cond and
 * uncond attention of one step, the head groups of a long sequence) and
 * order those streams themselves with events. No reference counterpart. */
int iris_b200_use_stream(void *cuda_stream);
void *iris_b200_stream(void);

/* CUDA-event stopwatch on the library's stream: start() records an event,
 * stop_ms() records a second one, waits for it and returns the elapsed
 * device time in milliseconds (< 0 on error). */
int iris_b200_timer_start(void);
float iris_b200_timer_stop_ms(void);

/* Numbered timing marks (0 <= id < 8192): mark() records a CUDA event on the
 * library's stream, mark_elapsed_ms() waits for `to` and returns the device
 * time between two recorded marks (< 0 on error). Lets a caller time single
 * kernels inside a longer region without leaving the stream. */
int iris_b200_mark(int id);
float iris_b200_mark_elapsed_ms(int from, int to);

/* Number of kernel launches the library has enqueued since init. */
unsigned long long iris_b200_launch_count(void);

/* ---- stream-ordered copies ------------------------------------------------ */

/* iris_dev_upload / iris_dev_download (iris_dev.h) block, as the reference's
 * do (iris_cuda.cu:191-230). These return at once: the copy runs on
 * `cuda_stream` (NULL: the library's stream) between page-locked host memory
 * and the device. A host overlaps the upload of step i + 1 and the download
 * of step i - 1 with the kernels of step i by giving the copies two streams of
 * their own and ordering them against the library's stream with events; the
 * helpers below let a plain-C host do that without CUDA headers. */
int iris_b200_upload_async(void *dst, const void *src, size_t bytes, void *cuda_stream);
int iris_b200_download_async(void *dst, const void *src, size_t bytes, void *cuda_stream);
void *iris_b200_host_alloc(size_t bytes);            /* page-locked host memory */
void iris_b200_host_free(void *p);
void *iris_b200_stream_create(void);
void iris_b200_stream_destroy(void *cuda_stream);
void *iris_b200_event_create(void);
void iris_b200_event_destroy(void *event);
int iris_b200_event_record(void *event, void *cuda_stream);        /* NULL stream: the library's */
int iris_b200_stream_wait_event(void *cuda_stream, void *event);   /* NULL stream: the library's */
int iris_b200_stream_sync(void *cuda_stream);

/* ---- prologue ----------------------------------------------------------- */

/* Q and K of one stream in a single launch: the two
 * iris_dev_head_norm_rope() calls every transformer block issues back to
 * back (iris_transformer_flux.c:3796-3801, :3834-3837;
 * iris_transformer_flux3.c:693-694; iris_transformer_zimage.c:1948-1949).
 * q and k share ld and the RoPE rows; wq / wk: [head_dim]. */
int iris_b200_qk_norm_rope(uint16_t *q, uint16_t *k, int ld,
                           const float *wq, const float *wk,
                           const float *rope_cos, const float *rope_sin,
                           int seq, int heads, int head_dim, float eps, int split_half);

/* The QKV projection with the prologue as its epilogue: the reference's
 * iris_dev_linear_bf16 (iris_cuda.cu:463-506, declared in iris_dev.h) and the
 * two iris_dev_head_norm_rope calls that follow it in every transformer block
 * (iris_transformer_flux.c:3795-3801 double blocks, :3832-3837 single blocks)
 * as ONE tcgen05 GEMM: y [rows, out] (row stride ldy) = x [rows, in] . W [out,
 * in]^T, bf16 in, fp32 accumulation, bf16 out; the column blocks [0, heads *
 * 128) (Q) and [heads * 128, 2 * heads * 128) (K) leave the kernel already
 * normalised per head (wq / wk [128], eps) and rotated (rope_cos / rope_sin
 * [rows, 64], consecutive pairs); all other columns (V, and the MLP half of a
 * single block's fused projection) are the plain product. Each Q / K value is
 * computed from the bf16-rounded product, as in the reference's two-kernel
 * sequence. Operands 16-byte aligned; in, out, ldy multiples of 8. */
int iris_b200_linear_qk_norm_rope(uint16_t *y, int ldy, const uint16_t *x, const uint16_t *W,
                                  int rows, int in, int out, int heads,
                                  const float *wq, const float *wk,
                                  const float *rope_cos, const float *rope_sin, float eps);

/* A block's input projection with the prologue AND SwiGLU as its epilogue: W
 * [3 * heads * 128 + 2 * mlp, in] holds the Q, K, V rows, then mlp gate rows,
 * then mlp up rows (the single blocks' fused weight,
 * iris_transformer_flux.c:3832-3842; with heads == 0 the gate | up weight of a
 * double block's feed-forward, :3818-3820). qkv [rows, 3 * heads * 128] (row
 * stride ldq) receives Q and K normalised and rotated and V, as
 * iris_b200_linear_qk_norm_rope stores them; act [rows, mlp] (row stride lda)
 * receives silu(gate) * up, gate and up rounded to bf16 first as the
 * reference's GEMM stores them before its k_swiglu (iris_cuda.cu:300-307).
 * One GEMM column tile pairs 128 gate columns with their 128 up columns (two
 * TMA boxes), so the [rows, 2 mlp] intermediate never exists. qkv may be NULL
 * when heads == 0. mlp a multiple of 8; operands 16-byte aligned. */
int iris_b200_linear_glu(uint16_t *qkv, int ldq, uint16_t *act, int lda,
                         const uint16_t *x, const uint16_t *W,
                         int rows, int in, int heads, int mlp,
                         const float *wq, const float *wk,
                         const float *rope_cos, const float *rope_sin, float eps);

/* The linear layers run as pairs of CTAs on 256 x 256 tiles
 * (tcgen05.mma.cta_group::2: each CTA stages half of the W tile, a third less
 * shared-memory traffic per SM) unless this is switched off, which leaves
 * single CTAs on 128 x 256 tiles (same results to the bit). enable: 1 on
 * (the default), 0 off, negative: only report. Returns the previous setting.
 * The row-parallel scatter mode always runs single CTAs. */
int iris_b200_linear_cta_pairs(int enable);

/* How a linear-layer launch cuts its work, as host arithmetic (for schedulers
 * and tests; nothing is launched): rows [0, split) and [split, rows) are the
 * two row groups (split == rows: one), `out` ordinary output columns followed
 * by glu_cols gate|up column pairs. Returns the number of 128 x 256 tiles, or
 * -1 for bad arguments, and writes the tile counts and the column-band width
 * of the work list. order (may be NULL): for the first `cap` work items, in
 * the order the persistent grid takes them, {first row, end of the row group,
 * column tile, 1 if a gate|up tile}. */
int iris_b200_linear_plan(int rows, int split, int in, int out, int glu_cols, int sm_count,
                          int *tiles_m, int *tiles_n, int *band_n, int *order, int cap);

/* The output projection with the gated residual as its epilogue: the
 * reference's iris_dev_linear_f32 followed by iris_dev_residual
 * (iris_transformer_flux.c:3843-3844 single blocks, :3809-3811 and :3821-3822
 * double blocks) as ONE tcgen05 GEMM: x_rows [rows, out] (fp32, row stride ldx)
 * += gate[c] * (a [rows, in] (bf16, row stride lda) . W [out, in]^T (row
 * stride ldw)), gate NULL meaning 1. The product is accumulated in fp32 and
 * never rounded, as in the reference's two-call sequence. Operands 16-byte
 * aligned; in, out, lda, ldw multiples of 8, ldx a multiple of 4. */
int iris_b200_linear_residual(float *x_rows, int ldx, const uint16_t *a, int lda,
                              const uint16_t *W, int ldw, const float *gate,
                              int rows, int in, int out);

/* ---- one single-stream block --------------------------------------------- */

/* Device bytes iris_b200_single_block() needs at `scratch` (256-byte aligned). */
size_t iris_b200_single_block_scratch_bytes(int seq, int dim, int mlp);

/* One FLUX.2 single-stream block on the device-resident fp32 hidden state x
 * [seq, dim], in place: what the reference issues per block in its device
 * forward (iris_transformer_flux.c:3828-3845; CPU form single_block_forward,
 * :3341-3477) - LayerNorm with (shift, scale), the fused QKV+MLP projection
 * with the Q/K prologue, joint attention over all rows, SwiGLU, the output
 * projection over [attention | mlp] and the gated residual - in four launches
 * (SwiGLU is part of the projection's epilogue).
 * w_in [3 dim + 2 mlp, dim], w_out [dim, dim + mlp]: bf16, as the checkpoints
 * store them. norm_q / norm_k [128]. mod = shift | scale | gate, [3 dim]
 * (the reference's mod_single). rope_cos / rope_sin [seq, 64]. key_mask: NULL
 * or [seq], nonzero = attend. head_dim is 128: dim == heads * 128. */
int iris_b200_single_block(float *x, void *scratch,
                           const uint16_t *w_in, const uint16_t *w_out,
                           const float *norm_q, const float *norm_k, const float *mod,
                           const float *rope_cos, const float *rope_sin,
                           int seq, int dim, int heads, int mlp, const int *key_mask);

/* A run of consecutive rows that share one modulation vector mod [3 dim] =
 * shift | scale | gate: the reference's f3_segment_t
 * (iris_transformer_flux3.c:118-121). */
typedef struct iris_b200_segment {
    int start, len;
    const float *mod;
} iris_b200_segment;

/* iris_b200_single_block with the rows in up to four segments, each with its
 * own modulation, and the norm epsilon as an argument: one FLUX.3 block as the
 * reference's dev_block_forward issues it (iris_transformer_flux3.c:680-703;
 * CPU form block_forward, :371-417), where text, image and reference-image rows
 * are modulated separately but share the weights. The segments must follow
 * one another and cover [0, seq). The gate of the residual is picked per row
 * inside the output projection's epilogue; LayerNorm picks shift and scale per
 * row. Four launches, like the single block. */
int iris_b200_single_block_segments(float *x, void *scratch,
                                    const uint16_t *w_in, const uint16_t *w_out,
                                    const float *norm_q, const float *norm_k,
                                    const iris_b200_segment *segs, int nsegs,
                                    const float *rope_cos, const float *rope_sin,
                                    int seq, int dim, int heads, int mlp, float eps,
                                    const int *key_mask);

/* ---- one single-stream block, tensor parallel ------------------------------ */

size_t iris_b200_single_block_tp_scratch_bytes(int seq, int heads_local, int mlp_local);

/* iris_b200_single_block over the group of iris_b200_ring_init, one process
 * per GPU (the reference is single device, iris_cuda.cu:122): the hidden state
 * is sharded by rows (rank r owns rows_of[r] consecutive rows; x_rows is this
 * rank's block, updated in place), the weights by heads and MLP columns: w_in
 * [3 * heads_local * 128 + 2 * mlp_local, dim] holds this rank's Q, K and V
 * head rows, then its gate rows, then its up rows; w_out [dim, heads_local *
 * 128 + mlp_local] the matching columns of the output projection. Both
 * collectives live inside kernels: LayerNorm stores this rank's normalised
 * rows into every rank's buffer over NVLink (the all-gather) and the input
 * projection waits, row tile by row tile, for the arrival words of the rows'
 * owners; the output projection's epilogue sends its fp32 partial sums to the
 * rows' owners (the reduce-scatter, iris_b200_outproj_residual), which apply
 * the gated residual. Five launches per block and rank; no NCCL call after
 * set-up; every wait is bounded (IRIS_B200_ETIMEOUT). rope tables [seq, 64]
 * cover all rows; mod = shift | scale | gate [3 dim]. Collective: every rank of
 * the group makes the same sequence of calls, within the wait limit
 * (iris_b200_set_wait_limit_us, 1 s by default) of one another: a rank whose
 * peers do not show up returns IRIS_B200_ETIMEOUT instead of waiting. */
int iris_b200_single_block_tp(float *x_rows, void *scratch,
                              const uint16_t *w_in, const uint16_t *w_out,
                              const float *norm_q, const float *norm_k, const float *mod,
                              const float *rope_cos, const float *rope_sin,
                              const int *rows_of, int dim, int heads_local, int mlp_local,
                              const int *key_mask);

/* ---- one double-stream block --------------------------------------------- */

/* The weights of one stream (text or image) of a double block, bf16 as the
 * checkpoints store them; the reference's device copy is dev_stream_flux_t
 * (iris_transformer_flux.c:3491-3494). */
typedef struct iris_b200_stream_weights {
    const uint16_t *qkv;      /* [3 dim, dim]: the Q, K and V rows */
    const uint16_t *proj;     /* [dim, dim] */
    const uint16_t *ff_in;    /* [2 mlp, dim]: the gate rows, then the up rows */
    const uint16_t *ff_out;   /* [dim, mlp] */
    const float *norm_q;      /* [128] */
    const float *norm_k;      /* [128] */
    const float *mod;         /* [6 dim]: shift1 scale1 gate1 shift2 scale2 gate2 */
} iris_b200_stream_weights;

size_t iris_b200_double_block_scratch_bytes(int seq, int dim, int mlp);

/* One FLUX.2 double-stream block on the device-resident fp32 hidden state x
 * [seq, dim] = [TEXT rows | IMAGE rows], in place: what the reference issues
 * per block in its device forward (iris_transformer_flux.c:3781-3823; CPU form
 * double_block_forward, :2133-2327). Per stream: LayerNorm with (shift1,
 * scale1), QKV projection with the Q/K prologue into the joint attention
 * input; joint attention over all rows; per stream: output projection with
 * the gate1 residual, LayerNorm with (shift2, scale2), the gate|up projection,
 * with SwiGLU in its epilogue, the down projection with the gate2 residual.
 * Seven launches: each covers both streams (two row groups with their own weights).
 * txt_seq: the number of text rows. rope tables [seq, 64] in row order.
 * key_mask: NULL or [seq]. head_dim is 128. */
int iris_b200_double_block(float *x, void *scratch,
                           const iris_b200_stream_weights *txt,
                           const iris_b200_stream_weights *img,
                           const float *rope_cos, const float *rope_sin,
                           int seq, int txt_seq, int dim, int heads, int mlp,
                           const int *key_mask);

/* ---- one Z-Image block --------------------------------------------------- */

/* The weights of one Z-Image (S3-DiT) block, bf16 matrices as the checkpoints
 * store them: the reference's zi_dev_block_t
 * (iris_transformer_zimage.c:1693-1697). */
typedef struct iris_b200_zimage_weights {
    const uint16_t *qkv;       /* [3 dim, dim] */
    const uint16_t *proj;      /* [dim, dim] */
    const uint16_t *ff_in;     /* [2 ff, dim]: the gate (w1) rows, then the up (w3) rows */
    const uint16_t *ff_out;    /* [dim, ff] (w2) */
    const float *norm_q;       /* [128] */
    const float *norm_k;       /* [128] */
    const float *attn_norm1, *attn_norm2, *ffn_norm1, *ffn_norm2;   /* [dim] */
} iris_b200_zimage_weights;

size_t iris_b200_zimage_block_scratch_bytes(int seq, int dim, int ff);

/* One Z-Image block on the device-resident fp32 hidden state x [seq, dim], in
 * place: what the reference's zi_dev_block issues
 * (iris_transformer_zimage.c:1940-1959; CPU form zi_block_forward, :801-880):
 * RMSNorm with (1 + scale_msa), QKV projection with the Q/K prologue,
 * attention under the key mask, output projection, x += tanh(gate_msa) *
 * RMSNorm(result), then the same around the SwiGLU feed-forward. Nine
 * launches for the reference's twelve calls. mod [4 dim] = scale_msa |
 * gate_msa | scale_mlp | gate_mlp, or NULL for the unmodulated context
 * refiner blocks. The norm epsilon is the reference's 1e-5. head_dim is 128. */
int iris_b200_zimage_block(float *x, void *scratch, const iris_b200_zimage_weights *w,
                           const float *mod, const float *rope_cos, const float *rope_sin,
                           int seq, int dim, int heads, int ff, const int *key_mask);

/* ---- attention ---------------------------------------------------------- */

enum {
    IRIS_B200_KERNEL_AUTO = 0,     /* what iris_dev_attention() picks */
    IRIS_B200_KERNEL_TCGEN05 = 1,  /* sm_100a TMA + tcgen05 kernel, or EUNSUPPORTED */
    IRIS_B200_KERNEL_GENERIC = 2   /* CUDA-core kernel covering every argument domain */
};

/* iris_dev_attention() with an explicit kernel choice and a status. */
int iris_b200_attention_ex(uint16_t *out, int ldo,
                           const uint16_t *q, const uint16_t *k, const uint16_t *v,
                           int ldi, int seq_q, int seq_k, int heads, int kv_heads,
                           int head_dim, float scale, int causal,
                           const int *key_mask, int kernel);

/* Which kernel AUTO would run for these arguments (one of the enum above). */
int iris_b200_attention_kernel_for(const void *out, int ldo, const void *q, const void *k,
                                   const void *v, int ldi, int heads, int kv_heads,
                                   int head_dim, int causal);

/* ---- multi-GPU decompositions (one process per GPU) ------------------------ */

/* Heads [first, first + count) of rank `rank` when `heads` are split over
 * `nranks`: the first heads % nranks ranks take one head more (30 heads over
 * 8 ranks: 4 4 4 4 4 4 3 3). A rank then runs the ordinary attention on the
 * column slice [first * head_dim, (first + count) * head_dim) of q, k, v and
 * out: heads are independent, nothing is exchanged. */
int iris_b200_head_shard(int heads, int nranks, int rank, int *first, int *count);

/* Classifier-free guidance runs `batch` independent passes over the same
 * image tokens (cond / uncond, iris_sample.c:698-712 in the reference runs
 * them one after the other). The ranks form min(batch, nranks) groups; rank
 * `rank` takes the entries first_entry, first_entry + entry_stride, ... and,
 * inside its group, the heads [first_head, first_head + head_count). */
int iris_b200_cfg_shard(int batch, int heads, int nranks, int rank,
                        int *first_entry, int *entry_stride, int *first_head, int *head_count);

/* Token rows [first, first + count) of a rank under sequence parallelism. */
int iris_b200_seq_shard(int seq, int nranks, int rank, int *first, int *count);

/* Rank whose K/V chunk is resident on `rank` at ring step `step`. */
int iris_b200_ring_source(int rank, int step, int nranks);

/* Key parts of one ring call: the attention launch of a call orders its work
 * by groups of ring steps, group i = steps [first_step[i], first_step[i] +
 * step_count[i]) (arrays of nranks entries), so that chunks are worked on in
 * the order they arrive. max_parts <= 0: the library's choice (up to four).
 * Returns the number of groups, -1 on bad arguments. Pure host arithmetic. */
int iris_b200_ring_plan(int nranks, int max_parts, int *first_step, int *step_count);

/* Attention of seq_q queries over ONE chunk of seq_k keys, merged into a
 * state carried between chunks: o_state [seq_q, heads * 128] fp32 (the
 * normalised output over the keys seen so far) and lse_state [heads, seq_q]
 * fp32 (their log2-sum-exp). first: the state is written, not read. last:
 * the merged result is written to `out` as bf16 and the state is left as it
 * is. first && last is the plain attention (state may be NULL). q has row
 * stride ldq, k and v share ldkv. tcgen05 kernel domain only (head_dim 128,
 * aligned views); key_mask covers this chunk's keys. Split-K over several
 * launches on one GPU. */
int iris_b200_attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                              const uint16_t *k, const uint16_t *v, int ldkv,
                              int seq_q, int seq_k, int heads, float scale,
                              const int *key_mask, float *o_state, float *lse_state,
                              int first, int last);

/* Attention whose keys are runs of rows taken from two K/V buffers
 * ("views"), in the order given: one launch, as if the runs were one
 * contiguous sequence. A run may be guarded by an arrival word: 32-bit words
 * in device memory that somebody else (a copy engine, another GPU, another
 * stream) advances once the run's rows are in place; the kernel waits, with
 * the library's wait limit, until (int)(word - arrive_value) >= 0 before it
 * loads the first row of the run. This is the attention of a ring call (own
 * rows, then the slots the peers fill) and of any host that streams K/V in.
 * nparts: 0 lets the library decide how to cut the keys of a query block
 * into separately scheduled parts, 1 forbids it, 2..8 asks for that many
 * parts of whole runs. tcgen05 kernel domain only; at most 16 runs; arrival
 * word indices below 32. */
typedef struct {
    int view;       /* 0: (k0, v0, ld0), 1: (k1, v1, ld1) */
    int row0, rows; /* key rows [row0, row0 + rows) of that view */
    int arrive;     /* index of the (first) arrival word guarding the run, -1: none */
    int rows_per_word; /* 0: one word guards the whole run; > 0: consecutive words guard this many rows each */
} iris_b200_key_run;
int iris_b200_attention_runs(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                             int seq_q, int heads, float scale,
                             const uint16_t *k0, const uint16_t *v0, int ld0,
                             const uint16_t *k1, const uint16_t *v1, int ld1,
                             const iris_b200_key_run *runs, int nruns,
                             const uint32_t *arrive_words, uint32_t arrive_value, int nparts);

/* Pure host arithmetic, for schedulers and tests: how a launch over these runs
 * cuts the keys of a query block into parts on a device with sm_count SMs.
 * part_tile (nparts + 1 entries, room for 9): part i covers the 128-key tiles
 * [part_tile[i], part_tile[i + 1]); *nkv: tiles over all runs. Returns the
 * number of parts, -1 on bad arguments. */
int iris_b200_attention_runs_plan(const iris_b200_key_run *runs, int nruns, int seq_q, int heads, int nparts,
                                  int sm_count, int *part_tile, int *nkv);

/* The same for the attention launch of one rank's ring call (copy-engine
 * transport): fills runs (room for 16) with "own rows, then the slots in ring
 * order" and part_tile with the groups of iris_b200_ring_plan() as tiles.
 * Returns runs * 100 + parts, -1 on bad arguments. */
int iris_b200_ring_launch_plan(int rank, int nranks, const int *rows_of, int heads, int max_parts, int sm_count,
                               iris_b200_key_run *runs, int *part_tile, int *nkv);

/* Ring sequence parallelism. One rank calls ring_unique_id(), the 128-byte id
 * is handed to every rank by the caller's own means, then every rank calls
 * ring_init() (NCCL, loaded at run time, carries the set-up exchanges).
 * ring_attention(): q, k, v are this rank's token rows (rows_of[rank] of
 * them, row stride ldi), rows_of lists the row count of every rank; out
 * receives the attention of the local queries over the keys of ALL ranks.
 * The chunk of step s is that of rank (rank - s) mod nranks; its owner's copy
 * engines push it straight into this GPU's slot s (pools mapped through CUDA
 * IPC) and then advance the slot's arrival word. The attention is one launch
 * over the runs "own rows, slot 1, ..., slot nranks - 1" that waits for each
 * arrival word inside the kernel, bounded by the wait limit: a peer that
 * never delivers ends the call with IRIS_B200_ETIMEOUT (reported by
 * iris_b200_check_device_status) instead of a hang. A received chunk is in
 * this GPU's memory before any kernel reads it. Without peer access the
 * chunks travel by ncclSend / ncclRecv and the launch follows them. Up to 16
 * ranks.
 * After any failure inside a call (an error return, or ETIMEOUT) the ring is
 * unusable: further calls return IRIS_B200_ECOMM until ring_destroy() and a
 * new ring_init() on every rank. Argument errors detected before anything is
 * enqueued leave it usable.
 * ring_configure() (before ring_init, same values on every rank): transport 0
 * = copy engines when possible, 1 = NCCL send/recv; parts = key parts of the
 * launch (0: the library's choice). ring_transport(): what is in use after the
 * first call (0 / 1, -1 before). */
int iris_b200_ring_unique_id(void *id128);
int iris_b200_ring_configure(int transport, int parts);
int iris_b200_ring_init(int rank, int nranks, const void *id128);
int iris_b200_ring_attention(uint16_t *out, int ldo,
                             const uint16_t *q, const uint16_t *k, const uint16_t *v,
                             int ldi, const int *rows_of, int heads, float scale);
int iris_b200_ring_transport(void);
void iris_b200_ring_destroy(void);

/* Device timeline of the last ring call, for measurement: with tracing on,
 * ring_timeline() waits for the device and fills ms[] with the times, in
 * milliseconds after the call's start on the library's stream, of: the
 * attention launch's start, its end, then the completion of the push of step
 * 1, 2, ... (copy-engine transport). Returns the number of entries. */
int iris_b200_ring_trace(int enable);
int iris_b200_ring_timeline(float *ms, int cap);

/* The out-projection after head-parallel attention, with its gated residual
 * and the reduction across ranks in one pass. The reference runs
 * iris_dev_linear_f32 + iris_dev_residual on one GPU
 * (iris_transformer_flux.c:3811-3812, 3841-3842; iris_cuda.cu:339-343). Here
 * rank r holds the k columns of the attention output that belong to its heads
 * (cat [seq, k] bf16, row stride ldc, all seq = sum(rows_of) rows) and the
 * matching k columns of the projection weights (W points at column k0 of the
 * row-major [dim, dim_in] matrix, row stride ldw). Its tcgen05 GEMM produces
 * fp32 partial sums for all rows; the epilogue stores every tile row straight
 * into the staging slab of the rank that owns the row (plain stores over
 * NVLink, rows_of[q] rows belong to rank q), and the owner adds
 * x_rows [rows_of[rank], dim] += gate [dim] * (sum over ranks) once every
 * rank's arrival word has come (bounded wait, IRIS_B200_ETIMEOUT otherwise;
 * gate NULL: plain sum). A reduce-scatter fused into the GEMM: no collective
 * library call and no separate pass over the partial sums. Needs the group of
 * iris_b200_ring_init() (one rank is allowed) and peer access between the
 * GPUs; dim a multiple of 8, k of 8, pointers 16-byte aligned. Collective:
 * every rank calls it with the same rows_of and dim. */
int iris_b200_outproj_residual(float *x_rows, const uint16_t *cat, int ldc, const uint16_t *W, int ldw,
                               const float *gate, const int *rows_of, int k, int dim);

/* The ring protocol on host threads (no device): one thread per rank and
 * memcpy in place of the copy engines, the same slots, pool sets, arrival
 * words, ring order and bounded waits as ring_attention(); the consumer
 * checks each received chunk (call number, row count, checksum) instead of
 * computing attention and folds it into a digest. For tests of the failure
 * paths that must not be provoked on a GPU: `faults` are injected on the host
 * and every rank comes back with a status, never blocking: IRIS_B200_ETIMEOUT
 * for a chunk that does not arrive within wait_limit_us, IRIS_B200_EPROTO for
 * one that arrives with the wrong call number, row count or content.
 * status / digest / calls_done: one entry per rank (calls_done: calls the rank
 * completed). ring_loopback_digest(): what a rank's digest must be after
 * `calls` fault-free calls. */
enum {
    IRIS_B200_LOOP_DROP = 1,      /* rank's push of (call, step) never happens */
    IRIS_B200_LOOP_DELAY = 2,     /* it happens delay_us later */
    IRIS_B200_LOOP_CORRUPT = 3,   /* a byte of the pushed rows is flipped */
    IRIS_B200_LOOP_LEAVE = 4,     /* the rank stops before `call` (step ignored) */
    IRIS_B200_LOOP_BAD_ROWS = 5   /* the pushed header announces one row too many */
};
typedef struct {
    int kind, rank, call, step;   /* calls count from 1; step < 0: every step */
    unsigned int delay_us;
} iris_b200_loop_fault;
int iris_b200_ring_loopback(int nranks, const int *rows_of, int row_bytes, int calls,
                            unsigned int wait_limit_us, const iris_b200_loop_fault *faults, int nfaults,
                            int *status_of_rank, uint64_t *digest_of_rank, int *calls_done_of_rank);
uint64_t iris_b200_ring_loopback_digest(int nranks, const int *rows_of, int row_bytes, int calls, int rank);

/* ---- attention without any allocation --------------------------------------- */

/* No counterpart in the reference. Split-K attention (the keys are walked in
 * `nsplit` chunks whose partial results are merged through a carried state)
 * for callers that are not allowed to allocate device memory where they run
 * attention: threads with real-time deadlines that must stay off the
 * driver's allocator lock, hosts that gave away their whole memory budget at
 * start-up. The carried state lives in a fixed 16.1 MiB array inside the
 * library image (held on every GPU that loads the library until exit), so
 * the call performs no cudaMalloc / cudaFree and calls no allocating routine.
 *
 * Limits: seq_q * heads * 128 <= iris_b200_attention_noalloc_max_elems()
 * (4 Mi), else IRIS_B200_EINVAL with a message; tcgen05 kernel domain only
 * (head_dim 128, heads == kv_heads, non-causal, aligned views, no key mask).
 * The first call on a device looks up the array's device address; make that
 * call before any stream capture. All calls share the array: calls whose
 * kernels may overlap on the GPU race on it (calls on the library's one
 * stream are ordered, hence safe). */
int iris_b200_attention_noalloc(uint16_t *out, int ldo,
                                const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                int ldi, int seq_q, int seq_k, int heads, float scale,
                                int nsplit);
size_t iris_b200_attention_noalloc_max_elems(void);

#ifdef __cplusplus
}
#endif

#endif /* IRIS_B200_H */
