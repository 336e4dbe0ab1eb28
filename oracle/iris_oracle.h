/*
 * TEST INFRASTRUCTURE, not product code: a CPU restatement of the reference's
 * joint-attention path (prologue + attention) used only as the checker in
 * tests, in the smoke test and as the timed CPU baseline. Nothing the library
 * ships links or calls it.
 *
 * Parity of this restatement is pinned: tests compare every function against
 * the reference's own CPU code compiled from its sources (oracle/_ref) and
 * against golden vectors generated from that code (tests/golden).
 */
#ifndef IRIS_ORACLE_H
#define IRIS_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- seeded inputs (iris_kernels.c:47-104) ---- */
void orc_rng_seed(uint64_t seed);
float orc_random_uniform(void);
float orc_random_normal(void);
void orc_randn(float *out, size_t n);

/* ---- bf16 helpers (iris_cuda.cu:236-245) ---- */
uint16_t orc_f2bf(float f);
float orc_bf2f(uint16_t v);
void orc_f32_to_bf16(uint16_t *dst, const float *src, size_t n);
void orc_bf16_to_f32(float *dst, const uint16_t *src, size_t n);
void orc_round_bf16(float *x, size_t n);          /* x = f32(bf16(x)) */

/* ---- iris_kernels.h surface ---- */
float orc_fast_expf(float x);                                         /* iris_kernels.h:21-32 */
void orc_softmax(float *x, int rows, int cols);                       /* iris_kernels.c:611-633 */
void orc_attention(float *out, const float *Q, const float *K, const float *V,
                   int batch, int heads, int seq_q, int seq_k, int head_dim,
                   float scale);                                      /* iris_kernels.c:656-697 */
void orc_flash_attention(float *out, const float *Q, const float *K, const float *V,
                         int seq_q, int seq_k, int heads, int head_dim,
                         float scale);                                /* iris_kernels.c:722-991 */
void orc_apply_rope(float *x, const float *freqs, int batch, int seq,
                    int heads, int head_dim);                         /* iris_kernels.c:998-1024 */
void orc_compute_rope_freqs(float *freqs, const int *pos, int seq, int dim,
                            float theta);                             /* iris_kernels.c:1026-1038 */

/* ---- iris_dev.h surface, fp32 and bf16 flavours ---- */

/* Per-head RMSNorm then pair rotation on fp32 x[s, h*hd + d] (row stride ld),
 * the math of apply_qk_norm + apply_rope_2d (iris_transformer_flux.c:1289,
 * :952) == head_rms_norm + apply_rope (iris_transformer_flux3.c:172,:185)
 * == zi_qk_norm + zi_apply_rope (iris_transformer_zimage.c:680,:629).
 * rope_cos/sin: [seq, hd/2]. */
void orc_head_norm_rope_f32(float *x, int ld, const float *w,
                            const float *rope_cos, const float *rope_sin,
                            int seq, int heads, int head_dim, float eps, int split_half);

/* Same on bf16 storage: widen, fp32 math, one RNE rounding
 * (k_head_norm_rope, iris_cuda.cu:403-420). */
void orc_head_norm_rope_bf16(uint16_t *x, int ld, const float *w,
                             const float *rope_cos, const float *rope_sin,
                             int seq, int heads, int head_dim, float eps, int split_half);

/* Attention over strided fp32 [seq, heads*hd] views with the semantics of
 * iris_dev_attention (iris_dev.h:83-92; iris_cuda.cu:514-536, :878-937):
 * GQA (query head h uses kv head h / (heads / kv_heads)), causal limit,
 * key_mask (0 = ignored key), a row with no valid key yields 0. Computed
 * with a full fp32 score row per query and orc_fast_expf like the CPU path.
 * rows: optional list of query indices (nrows entries) to compute; out rows
 * for other queries are left untouched. NULL = all rows. nthreads <= 0: one
 * thread per online core (heads are split over threads, as the reference's
 * BLAS build does, iris_transformer_flux.c:1569-1579). */
void orc_dev_attention(float *out, int ldo, const float *q, const float *k, const float *v,
                       int ldi, int seq_q, int seq_k, int heads, int kv_heads, int head_dim,
                       float scale, int causal, const int *key_mask,
                       const int *rows, int nrows, int nthreads);

/* ---- RoPE table builders, compact [seq, hd/2] layout ---- */

/* FLUX.2: theta^(-2d/axis_dim), axes (T, H, W, L) of axis_dim dims each
 * (iris_transformer_flux.c:823-1013, compaction :3754-3757). */
void orc_flux_rope_text(float *cos_out, float *sin_out, int txt_seq, int axis_dim, float theta);
void orc_flux_rope_image(float *cos_out, float *sin_out, int ph, int pw, int axis_dim,
                         float theta, int t_offset);

/* FLUX.3: angles in double, image rows at (0, 0.5 r, 0.5 c, l), text at
 * (0, 0, 0, s), reference image i at l = -(i + 1)
 * (iris_transformer_flux3.c:282-333). Returns the total row count. */
int orc_f3_joint_rope(float *cos_out, float *sin_out, int txt_seq, int img_h, int img_w,
                      const int *ref_h, const int *ref_w, int num_refs,
                      int head_dim, float theta);

/* Z-Image: axes of 32/48/48 dims and 1024/512/512 table rows, theta 256,
 * out-of-range position = identity rotation
 * (iris_transformer_zimage.c:604-622, :1924-1938). pos: [seq, 3]. */
void orc_zi_rope(float *cos_out, float *sin_out, const int *pos, int seq, float theta);
/* Positions and key mask of the [IMAGE | CAPTION] sequence, padded to
 * multiples of 32 (iris_transformer_zimage.c:1966-1994). pos: [seq, 3],
 * mask: [seq]. Returns seq. */
int orc_zi_positions(int *pos, int *mask, int ht, int wt, int cap_seq);

/* ---- the operators either side of the path, and one single-stream block ---- */
/* LayerNorm without affine parameters, then (1 + scale) and shift; fp32 in,
 * bf16 out (k_layer_norm_mod, iris_cuda.cu:349-370). shift / scale may be NULL. */
void orc_layer_norm_mod(uint16_t *out, const float *x, const float *shift, const float *scale,
                        int rows, int dim, float eps);
/* silu(gate) * up on bf16 column slices (k_swiglu, iris_cuda.cu:300-307). */
void orc_swiglu(uint16_t *out, int ldo, const uint16_t *gate, const uint16_t *up, int ldi,
                int rows, int cols);
/* x += gate * a in fp32, gate NULL = 1 (k_residual, iris_cuda.cu:309-314). */
void orc_residual(float *x, const float *a, const float *gate, int rows, int dim);
/* y = x . W^T, bf16 operands, fp32 accumulation and result
 * (iris_dev_linear_f32, iris_cuda.cu:560-584). nthreads <= 0: all cores. */
void orc_linear(float *y, int ldy, const uint16_t *x, int ldx, const uint16_t *W, int ldw,
                int rows, int in, int out, int nthreads);
/* One FLUX.2 single-stream block in the arithmetic of the reference's device
 * forward (iris_transformer_flux.c:3828-3845), in place on x [seq, dim] fp32.
 * w_in [3 dim + 2 mlp, dim], w_out [dim, dim + mlp] bf16; mod = shift | scale
 * | gate; rope tables compact [seq, head_dim / 2]. */
int orc_single_block(float *x, const uint16_t *w_in, const uint16_t *w_out,
                     const float *norm_q, const float *norm_k, const float *mod,
                     const float *rope_cos, const float *rope_sin,
                     int seq, int dim, int heads, int mlp, const int *key_mask, int nthreads);

/* The same with the rows in segments (start, len) that carry their own
 * modulation seg_mod[i] [3 dim], and the norm epsilon as an argument: one
 * FLUX.3 block (iris_transformer_flux3.c:680-703). */
int orc_single_block_segments(float *x, const uint16_t *w_in, const uint16_t *w_out,
                              const float *norm_q, const float *norm_k,
                              const int *seg_start, const int *seg_len, const float *const *seg_mod, int nsegs,
                              const float *rope_cos, const float *rope_sin,
                              int seq, int dim, int heads, int mlp, float eps, const int *key_mask, int nthreads);

/* The weights of one stream of a double block (the reference's
 * dev_stream_flux_t, iris_transformer_flux.c:3491-3494, plus the stream's
 * modulation): qkv [3 dim, dim], proj [dim, dim], ff_in [2 mlp, dim] (gate
 * rows, then up rows), ff_out [dim, mlp] in bf16; norm_q / norm_k [head_dim];
 * mod [6 dim] = shift1 scale1 gate1 shift2 scale2 gate2. */
typedef struct {
    const uint16_t *qkv, *proj, *ff_in, *ff_out;
    const float *norm_q, *norm_k, *mod;
} orc_stream_weights;
/* One FLUX.2 double-stream block in the arithmetic of the reference's device
 * forward (iris_transformer_flux.c:3781-3823), in place on x [seq, dim] =
 * [text rows | image rows]. */
int orc_double_block(float *x, const orc_stream_weights *txt, const orc_stream_weights *img,
                     const float *rope_cos, const float *rope_sin,
                     int seq, int txt_seq, int dim, int heads, int mlp, const int *key_mask, int nthreads);

/* RMSNorm rows (k_rms_norm, iris_cuda.cu:372-386; k_rms_norm_residual,
 * :388-400). scale / gate may be NULL. */
void orc_rms_norm_mod(uint16_t *out, const float *x, const float *w, const float *scale,
                      int rows, int dim, float eps);
void orc_rms_norm_residual(float *x, const float *a, const float *w, const float *gate,
                           int rows, int dim, float eps);
/* The weights of one Z-Image block (the reference's zi_dev_block_t,
 * iris_transformer_zimage.c:1693-1697): bf16 matrices, fp32 norm weights. */
typedef struct {
    const uint16_t *qkv, *proj, *ff_in, *ff_out;
    const float *norm_q, *norm_k, *attn_norm1, *attn_norm2, *ffn_norm1, *ffn_norm2;
} orc_zimage_weights;
/* One Z-Image block in the arithmetic of zi_dev_block
 * (iris_transformer_zimage.c:1940-1959), in place on x [seq, dim]; norm
 * epsilon 1e-5. */
int orc_zimage_block(float *x, const orc_zimage_weights *w, const float *mod,
                     const float *rope_cos, const float *rope_sin,
                     int seq, int dim, int heads, int ff, const int *key_mask, int nthreads);

/* ---- comparison metrics ---- */
/* Per head over the listed rows (NULL = all): max |a - b| and cosine.
 * a, b: [seq, heads*hd] with row strides lda / ldb. Writes heads entries. */
void orc_compare_heads(const float *a, int lda, const float *b, int ldb, int seq, int heads,
                       int head_dim, const int *rows, int nrows,
                       float *max_abs, float *cosine);

#ifdef __cplusplus
}
#endif

#endif
