/*
 * Additions of the B200 implementation to the reference's operator surface.
 *
 * Nothing here has a counterpart in the reference unless a comment says
 * which reference code it stands in for: the reference is single device,
 * single stream and reports errors only on stderr. These entry points add a
 * status word, stream sharing, device-side timing, a one-launch Q+K
 * prologue, kernel selection for tests, and the multi-GPU decompositions of
 * the attention (head shards, CFG split, ring sequence parallelism).
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
    IRIS_B200_ECOMM = 7         /* collective transport (NCCL) failed */
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

/* Launch schedule of one ring call: launch i covers the steps
 * [first_step[i], first_step[i] + step_count[i]) (arrays of nranks entries).
 * even_rows: every rank holds the same number of rows. Returns the number of
 * launches, -1 on bad arguments. Pure host arithmetic. */
int iris_b200_ring_plan(int nranks, int even_rows, int *first_step, int *step_count);

/* Attention of seq_q queries over ONE chunk of seq_k keys, merged into a
 * state carried between chunks: o_state [seq_q, heads * 128] fp32 (the
 * normalised output over the keys seen so far) and lse_state [heads, seq_q]
 * fp32 (their log2-sum-exp). first: the state is written, not read. last:
 * the merged result is written to `out` as bf16 and the state is left as it
 * is. first && last is the plain attention (state may be NULL). q has row
 * stride ldq, k and v share ldkv. tcgen05 kernel domain only (head_dim 128,
 * aligned views); key_mask covers this chunk's keys. Used for split-K on one
 * GPU and for every step of the ring. */
int iris_b200_attention_chunk(uint16_t *out, int ldo, const uint16_t *q, int ldq,
                              const uint16_t *k, const uint16_t *v, int ldkv,
                              int seq_q, int seq_k, int heads, float scale,
                              const int *key_mask, float *o_state, float *lse_state,
                              int first, int last);

/* Ring sequence parallelism over NCCL (loaded at run time). One rank calls
 * ring_unique_id(), the 128-byte id is handed to every rank by the caller's
 * own means, then every rank calls ring_init(). ring_attention(): q, k, v are
 * this rank's token rows (rows_of[rank] of them, row stride ldi), rows_of
 * lists the row count of every rank; out receives the attention of the local
 * queries over the keys of ALL ranks. At step s a rank works on the chunk of
 * rank (rank - s) mod nranks, which its owner sends directly; all transfers
 * are queued on a second stream at the start and overlap the attention of
 * the earlier steps. A received chunk is in this GPU's memory before any
 * kernel reads it. Up to 16 ranks. */
int iris_b200_ring_unique_id(void *id128);
int iris_b200_ring_init(int rank, int nranks, const void *id128);
int iris_b200_ring_attention(uint16_t *out, int ldo,
                             const uint16_t *q, const uint16_t *k, const uint16_t *v,
                             int ldi, const int *rows_of, int heads, float scale);
void iris_b200_ring_destroy(void);

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

/* Diagnostics for kernel bring-up: runs the tcgen05 kernel and dumps, into
 * `debug` (device, fp32), the raw scores S = Q K^T of the first key tile of
 * every CTA ([ctas * 256, 128]) followed by (m, l) per row ([ctas * 256, 2])
 * and 512 words of device timestamps (cycle counts of CTA 0 per key tile,
 * then wall-clock milestones of the first and the last CTA), so `debug`
 * holds ctas * 256 * 130 + 512 floats; ctas = ceil(seq_q / 256) * heads.
 * desc_fields: NULL, or four words: the
 * shared memory descriptor fields {qk_sbo, v_lbo, v_sbo} in 16-byte units
 * and a mode (bit 0 skip the softmax arithmetic, bit 1 skip the PV MMAs,
 * bit 2 skip the QK MMAs; results are then meaningless, only time is; bit 3
 * leave out the S dump). */
int iris_b200_attention_diag(uint16_t *out, int ldo,
                             const uint16_t *q, const uint16_t *k, const uint16_t *v,
                             int ldi, int seq_q, int seq_k, int heads, float scale,
                             const int *key_mask, float *debug, const uint32_t *desc_fields);

#ifdef __cplusplus
}
#endif

#endif /* IRIS_B200_H */
