/*
 * Device-resident operator surface of the joint-attention path.
 *
 * Same names, argument meaning and error behaviour as the reference's GPU
 * API (iris_dev.h of antirez/iris.c), restricted to what the attention path
 * needs: the small runtime (init / alloc / upload / download / sync), the
 * bf16 cast, the fused per-head RMSNorm + RoPE prologue and the scaled
 * dot-product attention. A program written against the reference header
 * links against libiris_b200.so unchanged for these calls.
 *
 * Conventions (reference iris_dev.h:8-15):
 *  - tensors are plain device pointers, bf16 stored as uint16_t, row-major;
 *  - every operation is enqueued in order on one internal stream; results
 *    are visible to later operations, and to the host after
 *    iris_dev_download() or iris_dev_sync();
 *  - operations return void; a failure prints "iris_dev: ..." on stderr and
 *    the call returns without doing the work (reference iris_cuda.cu:108-111).
 *    iris_b200_last_error() (iris_b200.h) additionally keeps the status.
 *  - global state, one device, not thread-safe.
 */
#ifndef IRIS_DEV_H
#define IRIS_DEV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces iris_dev.h:27-31 (iris_cuda.cu:117-172). init returns 1 if a
 * usable sm_100 GPU was found; it is idempotent. */
int iris_dev_init(void);
int iris_dev_available(void);
const char *iris_dev_name(void);
void iris_dev_cleanup(void);

/* Replaces iris_dev.h:33-46 (iris_cuda.cu:174-230). alloc returns NULL on
 * failure and at least one byte for a zero size; free accepts NULL and
 * first waits for the stream; upload / download return after the copy, so
 * the host buffer can be reused. */
void *iris_dev_alloc(size_t bytes);
void iris_dev_free(void *p);
void iris_dev_upload(void *dst, const void *src, size_t bytes);
void iris_dev_download(void *dst, const void *src, size_t bytes);
void iris_dev_upload_2d(void *dst, size_t dst_stride, const void *src, size_t src_stride,
                        size_t row_bytes, size_t rows);
void iris_dev_sync(void);

/* dst[i] = bf16(src[i]), round to nearest even. Replaces iris_dev.h:48-49
 * (iris_cuda.cu:271-274). */
void iris_dev_f32_to_bf16(uint16_t *dst, const float *src, size_t n);

/* y [rows, out] = x [rows, in] . W [out, in]^T, bf16 operands and result, fp32
 * accumulation (row-major, W as the checkpoints store it). Replaces
 * iris_dev.h:52-53 (iris_cuda.cu:463-506, a cuBLAS call there; a tcgen05
 * kernel here). Operands 16-byte aligned, in and out multiples of 8. */
void iris_dev_linear_bf16(uint16_t *y, const uint16_t *x, const uint16_t *W,
                          int rows, int in, int out);

/* Same product with an fp32 result (iris_dev.h:50-51, iris_cuda.cu:560-584):
 * the output projections, whose result joins the fp32 hidden state. */
void iris_dev_linear_f32(float *y, const uint16_t *x, const uint16_t *W,
                         int rows, int in, int out);

/* out = LayerNorm(x) * (1 + scale) + shift without affine parameters, fp32
 * in, bf16 out; shift / scale: [dim], either may be NULL. Replaces
 * iris_dev.h:57-59 (kernel iris_cuda.cu:349-370): mean, then the variance
 * about the mean, both in fp32. */
void iris_dev_layer_norm_mod(uint16_t *out, const float *x,
                             const float *shift, const float *scale,
                             int rows, int dim, float eps);

/* out = RMSNorm(x) * w, and the same times (1 + scale) with scale [dim] or
 * NULL; fp32 in, bf16 out. Replace iris_dev.h:61-68 (kernel
 * iris_cuda.cu:372-386). */
void iris_dev_rms_norm(uint16_t *out, const float *x, const float *w,
                       int rows, int dim, float eps);
void iris_dev_rms_norm_mod(uint16_t *out, const float *x, const float *w,
                           const float *scale, int rows, int dim, float eps);

/* x += tanh(gate) * RMSNorm(a) * w in fp32; gate [dim] or NULL for an ungated
 * residual. Replaces iris_dev.h:70-73 (kernel iris_cuda.cu:388-400). */
void iris_dev_rms_norm_residual(float *x, const float *a, const float *w,
                                const float *gate, int rows, int dim, float eps);

/* out[r, c] = silu(gate[r, c]) * up[r, c] on bf16 column slices (gate / up row
 * stride ldi, out row stride ldo). Replaces iris_dev.h:94-95 (kernel
 * iris_cuda.cu:300-307). The exponential is the hardware approximation
 * (ex2.approx), so a result may differ from the reference's expf() by one
 * bf16 unit in the last place where it falls on a rounding boundary. */
void iris_dev_swiglu(uint16_t *out, int ldo, const uint16_t *gate,
                     const uint16_t *up, int ldi, int rows, int cols);

/* x[r, c] += gate[c] * a[r, c] in fp32, or x += a when gate is NULL. Replaces
 * iris_dev.h:98-99 (kernel iris_cuda.cu:309-314). */
void iris_dev_residual(float *x, const float *a, const float *gate,
                       int rows, int dim);

/* In place on the bf16 heads x[s, h * head_dim + d] (row stride ld, in
 * elements): per-head RMSNorm x * rsqrt(mean(x^2) + eps) * w[d], then
 * rotation of pair i by the angle of row s (rope_cos / rope_sin:
 * [seq, head_dim / 2], fp32). Pairs are consecutive (2i, 2i + 1), or
 * (i, i + head_dim / 2) when split_half is set. fp32 arithmetic, one
 * round-to-nearest-even at the store. Replaces iris_dev.h:74-81
 * (iris_cuda.cu:403-453). */
void iris_dev_head_norm_rope(uint16_t *x, int ld, const float *w,
                             const float *rope_cos, const float *rope_sin,
                             int seq, int heads, int head_dim, float eps,
                             int split_half);

/* Scaled dot-product attention over bf16 [seq, heads * head_dim] tensors.
 * q, k, v share the row stride ldi, out has row stride ldo (elements). With
 * fewer kv heads (GQA) query head h uses kv head h / (heads / kv_heads).
 * causal: query i ignores keys j > i. key_mask: device int [seq_k], 0 =
 * ignored key, or NULL. A query with no valid key gets a zero row.
 * Replaces iris_dev.h:83-92 (iris_cuda.cu:878-937). */
void iris_dev_attention(uint16_t *out, int ldo,
                        const uint16_t *q, const uint16_t *k, const uint16_t *v,
                        int ldi, int seq_q, int seq_k, int heads, int kv_heads,
                        int head_dim, float scale, int causal,
                        const int *key_mask);

#ifdef __cplusplus
}
#endif

#endif /* IRIS_DEV_H */
