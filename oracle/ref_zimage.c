/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * Exported wrappers around the `static` Z-Image prologue / attention helpers
 * of the reference, compiled from where the reference lies (Makefile REF).
 *
 * Reference functions reached (iris_transformer_zimage.c):
 *   zi_precompute_rope :604, zi_apply_rope :629, zi_qk_norm :680,
 *   zi_attention :698 (with identity projections, to pin the key-mask rule).
 */
#include "iris_transformer_zimage.c"

/* Timing accumulators the reference expects from iris_sample.c. */
double iris_timing_zi_total, iris_timing_zi_embeddings, iris_timing_zi_noise_refiner;
double iris_timing_zi_context_refiner, iris_timing_zi_main_blocks, iris_timing_zi_final;

static void zi_ctx(zi_transformer_t *tf, int heads, int head_dim) {
    memset(tf, 0, sizeof(*tf));
    tf->n_heads = heads;
    tf->head_dim = head_dim;
    tf->dim = heads * head_dim;
    tf->rope_theta = 256.0f;
    tf->axes_dims[0] = 32; tf->axes_dims[1] = 48; tf->axes_dims[2] = 48;
    tf->axes_lens[0] = 1024; tf->axes_lens[1] = 512; tf->axes_lens[2] = 512;
    zi_precompute_rope(tf);
}

static void zi_ctx_free(zi_transformer_t *tf) {
    for (int ax = 0; ax < 3; ax++) { free(tf->rope_cos[ax]); free(tf->rope_sin[ax]); }
}

void ref_zi_qk_norm(float *x, const float *w, int seq, int heads, int head_dim, float eps) {
    zi_qk_norm(x, w, seq, heads, head_dim, eps);
}

/* pos: [seq, 3] integer (T, H, W) positions. */
void ref_zi_apply_rope(float *x, const int *pos, int seq, int heads, int head_dim) {
    zi_transformer_t tf;
    zi_ctx(&tf, heads, head_dim);
    zi_apply_rope(x, pos, seq, heads, &tf);
    zi_ctx_free(&tf);
}

/* Whole zi_attention with identity q/k/v/out projections and unit norm
 * weights: out = SDPA(rope(norm(x)), rope(norm(x)), x) under `mask`
 * (int [seq], 0 = padding key, or NULL). Small head counts only: the
 * identity matrices are [dim, dim]. */
int ref_zi_attention_identity(float *out, const float *x, const int *pos, const int *mask,
                              int seq, int heads, int head_dim) {
    zi_transformer_t tf;
    zi_ctx(&tf, heads, head_dim);
    int dim = tf.dim;
    float *eye = calloc((size_t)dim * dim, sizeof(float));
    float *ones = malloc((size_t)head_dim * sizeof(float));
    tf.work_qkv = malloc((size_t)3 * seq * dim * sizeof(float));
    tf.work_attn = malloc((size_t)seq * seq * sizeof(float));
    if (!eye || !ones || !tf.work_qkv || !tf.work_attn) return -1;
    for (int i = 0; i < dim; i++) eye[(size_t)i * dim + i] = 1.0f;
    for (int i = 0; i < head_dim; i++) ones[i] = 1.0f;
    zi_block_t b;
    memset(&b, 0, sizeof(b));
    b.attn_q_weight = b.attn_k_weight = b.attn_v_weight = b.attn_out_weight = eye;
    b.attn_norm_q = b.attn_norm_k = ones;
    zi_attention(out, x, &b, pos, mask, seq, &tf);
    free(eye); free(ones); free(tf.work_qkv); free(tf.work_attn);
    zi_ctx_free(&tf);
    return 0;
}
