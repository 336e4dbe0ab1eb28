/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * Thin exported wrappers around the `static` FLUX.2 prologue / attention
 * helpers of the reference. The reference source is compiled where it lies
 * (include path given by the Makefile's REF variable); nothing of it is
 * copied here. The wrappers only forward arguments.
 *
 * Reference functions reached (iris_transformer_flux.c):
 *   apply_qk_norm :1289, compute_rope_2d :823, compute_rope_2d_with_t_offset
 *   :887, apply_rope_2d :952, compute_rope_text :981, mha_forward :1585,
 *   joint_attention :1682, ensure_attn_scores :1382, single_block_forward
 *   :3341, double_block_forward :2133.
 */
#include "iris_transformer_flux.c"

/* Timing accumulators the reference expects from iris_sample.c:29-58. */
double iris_timing_transformer_total, iris_timing_transformer_double;
double iris_timing_transformer_single, iris_timing_transformer_final;

void ref_flux_qk_norm(float *q, float *k, const float *qw, const float *kw,
                      int seq, int heads, int head_dim, float eps) {
    apply_qk_norm(q, k, qw, kw, seq, heads, head_dim, eps);
}

void ref_flux_rope_text(float *cos_out, float *sin_out, int txt_seq, int axis_dim, float theta) {
    compute_rope_text(cos_out, sin_out, txt_seq, axis_dim, theta);
}

void ref_flux_rope_2d(float *cos_out, float *sin_out, int ph, int pw, int axis_dim, float theta) {
    compute_rope_2d(cos_out, sin_out, ph, pw, axis_dim, theta);
}

void ref_flux_rope_2d_t(float *cos_out, float *sin_out, int ph, int pw, int axis_dim,
                        float theta, int t_offset) {
    compute_rope_2d_with_t_offset(cos_out, sin_out, ph, pw, axis_dim, theta, t_offset);
}

void ref_flux_apply_rope_2d(float *x, const float *cos_f, const float *sin_f,
                            int seq, int heads, int head_dim) {
    apply_rope_2d(x, cos_f, sin_f, seq, heads, head_dim, head_dim / 4);
}

static int flux_ctx(iris_transformer_flux_t *tf, int img_seq, int txt_seq, int heads, int head_dim) {
    memset(tf, 0, sizeof(*tf));
    tf->num_heads = heads;
    tf->head_dim = head_dim;
    tf->hidden_size = heads * head_dim;
    tf->axis_dim = head_dim / 4;
    tf->rope_theta = 2000.0f;
    size_t n = (size_t)(img_seq + txt_seq) * heads * head_dim;
    tf->attn_cat_k = malloc(n * sizeof(float));
    tf->attn_cat_v = malloc(n * sizeof(float));
    if (!tf->attn_cat_k || !tf->attn_cat_v) return -1;
    return ensure_attn_scores(tf, img_seq, txt_seq);
}

static void flux_ctx_free(iris_transformer_flux_t *tf) {
    free(tf->attn_cat_k);
    free(tf->attn_cat_v);
    free(tf->attn_scores);
}

/* Joint attention of a double block: K/V concatenated as [TEXT, IMAGE]. */
int ref_flux_joint_attention(float *img_out, float *txt_out,
                             const float *img_q, const float *img_k, const float *img_v,
                             const float *txt_q, const float *txt_k, const float *txt_v,
                             int img_seq, int txt_seq, int heads, int head_dim) {
    iris_transformer_flux_t tf;
    if (flux_ctx(&tf, img_seq, txt_seq, heads, head_dim) != 0) { flux_ctx_free(&tf); return -1; }
    joint_attention(img_out, txt_out, img_q, img_k, img_v, txt_q, txt_k, txt_v,
                    img_seq, txt_seq, heads, head_dim, &tf);
    flux_ctx_free(&tf);
    return 0;
}

/* Self attention of a single block over the already concatenated sequence. */
int ref_flux_mha(float *out, const float *q, const float *k, const float *v,
                 int seq, int heads, int head_dim) {
    iris_transformer_flux_t tf;
    if (flux_ctx(&tf, seq, 0, heads, head_dim) != 0) { flux_ctx_free(&tf); return -1; }
    mha_forward(out, q, k, v, seq, heads, head_dim, &tf);
    flux_ctx_free(&tf);
    return 0;
}

/* One single-stream block on the CPU, fp32 weights: single_block_forward with
 * a context that holds only the work buffers the function touches (the
 * reference allocates the same in its loader, :1443-1461). hidden [seq, dim]
 * is updated in place. t_emb [dim] and adaln_weight [3 dim, dim] give the
 * modulation as in the reference; rope tables are the reference's own
 * ([rows, head_dim]). Returns 0, or -1 when memory runs out. */
int ref_flux_single_block(float *hidden, const float *w_in, const float *w_out,
                          const float *norm_q, const float *norm_k,
                          const float *t_emb, const float *adaln_weight,
                          const float *img_cos, const float *img_sin,
                          const float *txt_cos, const float *txt_sin,
                          int seq, int img_offset, int heads, int head_dim, int mlp) {
    iris_transformer_flux_t tf;
    single_block_t block;
    if (flux_ctx(&tf, seq, 0, heads, head_dim) != 0) { flux_ctx_free(&tf); return -1; }
    int dim = heads * head_dim, fused = 3 * dim + 2 * mlp;
    size_t n = (size_t)seq;
    tf.mlp_hidden = mlp;
    tf.work1 = malloc(n * dim * sizeof(float));
    tf.work2 = malloc((n * fused + 3 * (size_t)dim) * sizeof(float));
    tf.single_q = malloc(n * dim * sizeof(float));
    tf.single_k = malloc(n * dim * sizeof(float));
    tf.single_v = malloc(n * dim * sizeof(float));
    tf.single_mlp_gate = malloc(n * mlp * sizeof(float));
    tf.single_mlp_up = malloc(n * mlp * sizeof(float));
    tf.single_attn_out = malloc(n * dim * sizeof(float));
    tf.single_concat = malloc(n * (dim + mlp) * sizeof(float));
    tf.t_emb_silu = malloc((size_t)dim * sizeof(float));
    int ok = tf.work1 && tf.work2 && tf.single_q && tf.single_k && tf.single_v && tf.single_mlp_gate &&
             tf.single_mlp_up && tf.single_attn_out && tf.single_concat && tf.t_emb_silu;
    if (ok) {
        memset(&block, 0, sizeof(block));
        block.qkv_mlp_weight = (float *)w_in;
        block.proj_mlp_weight = (float *)w_out;
        block.norm_q_weight = (float *)norm_q;
        block.norm_k_weight = (float *)norm_k;
        single_block_forward(hidden, &block, t_emb, adaln_weight, img_cos, img_sin, txt_cos, txt_sin,
                             seq, img_offset, &tf);
    }
    free(tf.work1); free(tf.work2); free(tf.single_q); free(tf.single_k); free(tf.single_v);
    free(tf.single_mlp_gate); free(tf.single_mlp_up); free(tf.single_attn_out); free(tf.single_concat);
    free(tf.t_emb_silu);
    flux_ctx_free(&tf);
    return ok ? 0 : -1;
}

/* One double-stream block on the CPU, fp32 weights: double_block_forward with
 * a context that holds only the work buffers it touches. w[9] per stream: Q,
 * K, V, proj [dim, dim], mlp gate, up [mlp, dim], down [dim, mlp], norm_q,
 * norm_k [head_dim]. mod [6 dim] per stream. Hidden states in place. */
int ref_flux_double_block(float *img_hidden, float *txt_hidden,
                          const float *const *img_w, const float *const *txt_w,
                          const float *img_mod, const float *txt_mod,
                          const float *img_cos, const float *img_sin,
                          const float *txt_cos, const float *txt_sin,
                          int img_seq, int txt_seq, int heads, int head_dim, int mlp) {
    iris_transformer_flux_t tf;
    double_block_t b;
    if (flux_ctx(&tf, img_seq, txt_seq, heads, head_dim) != 0) { flux_ctx_free(&tf); return -1; }
    int dim = heads * head_dim;
    size_t n = (size_t)img_seq + txt_seq;
    tf.mlp_hidden = mlp;
    tf.work1 = malloc(n * dim * sizeof(float));
    tf.work2 = malloc(3 * n * dim * sizeof(float));
    tf.ffn_gate = malloc(n * mlp * sizeof(float));
    tf.ffn_up = malloc(n * mlp * sizeof(float));
    tf.double_img_attn_out = malloc((size_t)img_seq * dim * sizeof(float));
    tf.double_txt_attn_out = malloc((size_t)txt_seq * dim * sizeof(float));
    int ok = tf.work1 && tf.work2 && tf.ffn_gate && tf.ffn_up && tf.double_img_attn_out && tf.double_txt_attn_out;
    if (ok) {
        memset(&b, 0, sizeof(b));
        b.img_q_weight = (float *)img_w[0]; b.img_k_weight = (float *)img_w[1]; b.img_v_weight = (float *)img_w[2];
        b.img_proj_weight = (float *)img_w[3];
        b.img_mlp_gate_weight = (float *)img_w[4]; b.img_mlp_up_weight = (float *)img_w[5];
        b.img_mlp_down_weight = (float *)img_w[6];
        b.img_norm_q_weight = (float *)img_w[7]; b.img_norm_k_weight = (float *)img_w[8];
        b.txt_q_weight = (float *)txt_w[0]; b.txt_k_weight = (float *)txt_w[1]; b.txt_v_weight = (float *)txt_w[2];
        b.txt_proj_weight = (float *)txt_w[3];
        b.txt_mlp_gate_weight = (float *)txt_w[4]; b.txt_mlp_up_weight = (float *)txt_w[5];
        b.txt_mlp_down_weight = (float *)txt_w[6];
        b.txt_norm_q_weight = (float *)txt_w[7]; b.txt_norm_k_weight = (float *)txt_w[8];
        double_block_forward(img_hidden, txt_hidden, &b, img_mod, txt_mod, img_cos, img_sin, txt_cos, txt_sin,
                             img_seq, txt_seq, &tf);
    }
    free(tf.work1); free(tf.work2); free(tf.ffn_gate); free(tf.ffn_up);
    free(tf.double_img_attn_out); free(tf.double_txt_attn_out);
    flux_ctx_free(&tf);
    return ok ? 0 : -1;
}

int ref_flux_attn_threads(int heads) {
#ifdef USE_BLAS
    return get_attn_num_threads(heads);
#else
    (void)heads;
    return 1;
#endif
}
