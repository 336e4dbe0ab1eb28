/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * Exported wrappers around the `static` Z-Image prologue / attention helpers
 * of the reference, compiled from where the reference lies (Makefile REF).
 *
 * Reference functions reached (iris_transformer_zimage.c):
 *   zi_precompute_rope :604, zi_apply_rope :629, zi_qk_norm :680,
 *   zi_attention :698 (with identity projections, to pin the key-mask rule),
 *   zi_ffn :775, zi_block_forward :801.
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

/* One Z-Image block on the CPU: zi_block_forward over x [seq, dim] in place.
 * w[11] (fp32): attn q, k, v, out [dim, dim]; ffn w1 (gate), w3 (up) [ff, dim],
 * w2 (down) [dim, ff]; attn_norm1, attn_norm2, ffn_norm1, ffn_norm2 [dim].
 * norm_q / norm_k [head_dim]. mod [4 dim] = scale_msa | gate_msa | scale_mlp |
 * gate_mlp, or NULL for an unmodulated block; it is handed to the reference as
 * the bias of a modulation layer whose weight is zero, so that the function
 * computes exactly these values. pos [seq, 3], mask [seq] or NULL. */
int ref_zi_block(float *x, const float *const *w, const float *norm_q, const float *norm_k,
                 const float *mod, const int *pos, const int *mask,
                 int seq, int heads, int head_dim, int ff) {
    zi_transformer_t tf;
    zi_block_t b;
    zi_ctx(&tf, heads, head_dim);
    int dim = tf.dim;
    size_t n = (size_t)seq * dim;
    tf.ffn_dim = ff;
    tf.adaln_dim = 1;
    tf.max_seq = seq;
    tf.work_tmp = malloc(4 * n * sizeof(float));
    tf.work_qkv = malloc(3 * n * sizeof(float));
    tf.work_attn = malloc((size_t)seq * seq * sizeof(float));
    tf.work_ffn = malloc((size_t)2 * seq * ff * sizeof(float));
    float *zero_w = calloc((size_t)4 * dim, sizeof(float));
    float t_emb = 0.0f;
    int ok = tf.work_tmp && tf.work_qkv && tf.work_attn && tf.work_ffn && zero_w;
    if (ok) {
        memset(&b, 0, sizeof(b));
        b.attn_q_weight = (float *)w[0]; b.attn_k_weight = (float *)w[1]; b.attn_v_weight = (float *)w[2];
        b.attn_out_weight = (float *)w[3];
        b.ffn_w1 = (float *)w[4]; b.ffn_w3 = (float *)w[5]; b.ffn_w2 = (float *)w[6];
        b.attn_norm1 = (float *)w[7]; b.attn_norm2 = (float *)w[8];
        b.ffn_norm1 = (float *)w[9]; b.ffn_norm2 = (float *)w[10];
        b.attn_norm_q = (float *)norm_q; b.attn_norm_k = (float *)norm_k;
        if (mod) {
            b.adaln_weight = zero_w;
            b.adaln_bias = (float *)mod;
        }
        zi_block_forward(x, &b, pos, mask, &t_emb, seq, &tf);
    }
    free(tf.work_tmp); free(tf.work_qkv); free(tf.work_attn); free(tf.work_ffn); free(zero_w);
    zi_ctx_free(&tf);
    return ok ? 0 : -1;
}
