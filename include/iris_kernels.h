/*
 * Host-pointer fp32 operator surface of the attention path.
 *
 * Same names and argument meaning as the attention / softmax / RoPE entry
 * points of the reference's CPU kernel header (iris_kernels.h of
 * antirez/iris.c). Every function takes HOST pointers; the work is done on
 * the GPU: upload, compute, download, all inside the call. There is no CPU
 * path: without an initialised device the call prints an error, records
 * IRIS_B200_ENODEV and leaves the output untouched.
 *
 * Precision: attention runs on bf16 operands with fp32 accumulation (max
 * abs error <= 2e-2 against the fp32 CPU result for unit-variance inputs);
 * softmax and RoPE run in fp32.
 */
#ifndef IRIS_KERNELS_H
#define IRIS_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Row softmax in place over x[rows, cols]. Replaces iris_kernels.h:158-159
 * (iris_kernels.c:611-646). */
void iris_softmax(float *x, int rows, int cols);
/* The same routine under the name the reference's BLAS attention variants
 * call (iris_kernels.h:159; iris_transformer_flux.c:1512, 1547, 1558). */
void iris_softmax_cpu(float *x, int rows, int cols);

/* Batched attention, Q/out: [batch, heads, seq_q, head_dim], K/V: [batch,
 * heads, seq_k, head_dim]. Replaces iris_kernels.h:173-175
 * (iris_kernels.c:656-697). */
void iris_attention(float *out, const float *Q, const float *K, const float *V,
                    int batch, int heads, int seq_q, int seq_k, int head_dim,
                    float scale);

/* Attention on the transformer layout, Q/out: [seq_q, heads * head_dim],
 * K/V: [seq_k, heads * head_dim]. Replaces iris_kernels.h:188-189
 * (iris_kernels.c:899-991). */
void iris_flash_attention(float *out, const float *Q, const float *K, const float *V,
                          int seq_q, int seq_k, int heads, int head_dim, float scale);

/* Split-half RoPE in place on x[batch, seq, heads, head_dim] with
 * freqs[seq, head_dim / 2, 2] = (cos, sin). Replaces iris_kernels.h:196-197
 * (iris_kernels.c:998-1024). */
void iris_apply_rope(float *x, const float *freqs,
                     int batch, int seq, int heads, int head_dim);

/* freqs[s, d] = (cos, sin)(pos[s] * theta^(-2d/dim)). Replaces
 * iris_kernels.h:204 (iris_kernels.c:1026-1038). */
void iris_compute_rope_freqs(float *freqs, const int *pos, int seq, int dim, float theta);

#ifdef __cplusplus
}
#endif

#endif /* IRIS_KERNELS_H */
