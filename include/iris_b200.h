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

/* Diagnostics for kernel bring-up: runs the tcgen05 kernel and dumps, into
 * `debug` (device, fp32), the raw scores S = Q K^T of the first key tile of
 * every CTA ([ctas * 256, 128]) followed by (m, l) per row ([ctas * 256, 2]);
 * ctas = ceil(seq_q / 256) * heads. desc_fields: NULL, or four words: the
 * shared memory descriptor fields {qk_sbo, v_lbo, v_sbo} in 16-byte units
 * and a mode (bit 0 skip the softmax arithmetic, bit 1 skip the PV MMAs,
 * bit 2 skip the QK MMAs; results are then meaningless, only time is). */
int iris_b200_attention_diag(uint16_t *out, int ldo,
                             const uint16_t *q, const uint16_t *k, const uint16_t *v,
                             int ldi, int seq_q, int seq_k, int heads, float scale,
                             const int *key_mask, float *debug, const uint32_t *desc_fields);

#ifdef __cplusplus
}
#endif

#endif /* IRIS_B200_H */
