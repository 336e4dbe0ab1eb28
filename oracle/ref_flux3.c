/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * Exported wrappers around the `static` FLUX.3 prologue / attention helpers
 * of the reference, compiled from where the reference lies (Makefile REF).
 *
 * Reference functions reached (iris_transformer_flux3.c):
 *   head_rms_norm :172, apply_rope :185, attention :204, rope_rows :282,
 *   image_positions :300, joint_rope :314, ensure_work :344,
 *   block_forward :371.
 */
#include "iris_transformer_flux3.c"

static void f3_ctx(iris_transformer_flux3_t *tf, int heads, int head_dim, float theta) {
    memset(tf, 0, sizeof(*tf));
    tf->heads = heads;
    tf->head_dim = head_dim;
    tf->dim = heads * head_dim;
    tf->rope_theta = theta;
    tf->eps = 1e-6f;
    for (int i = 0; i < F3_ROPE_AXES; i++) tf->axes_dim[i] = head_dim / F3_ROPE_AXES;
}

void ref_f3_head_rms_norm(float *x, const float *w, int seq, int heads, int head_dim, float eps) {
    head_rms_norm(x, w, seq, heads, head_dim, eps);
}

void ref_f3_apply_rope(float *x, const float *cos_t, const float *sin_t,
                       int seq, int heads, int head_dim) {
    apply_rope(x, cos_t, sin_t, seq, heads, head_dim);
}

/* cos_out / sin_out: caller buffers of [total, head_dim / 2]. Returns total. */
int ref_f3_joint_rope(float *cos_out, float *sin_out, int txt_seq, int img_h, int img_w,
                      const int *ref_h, const int *ref_w, int num_refs,
                      int heads, int head_dim, float theta) {
    iris_transformer_flux3_t tf;
    f3_ctx(&tf, heads, head_dim, theta);
    float *c = NULL, *s = NULL;
    joint_rope(&tf, txt_seq, img_h, img_w, ref_h, ref_w, num_refs, &c, &s);
    int total = txt_seq + img_h * img_w;
    for (int i = 0; i < num_refs; i++) total += ref_h[i] * ref_w[i];
    size_t n = (size_t)total * (head_dim / 2);
    memcpy(cos_out, c, n * sizeof(float));
    memcpy(sin_out, s, n * sizeof(float));
    free(c);
    free(s);
    return total;
}

int ref_f3_attention(float *out, const float *q, const float *k, const float *v,
                     int seq, int heads, int head_dim) {
    float *scores = malloc((size_t)F3_ATTN_QCHUNK * seq * sizeof(float));
    if (!scores) return -1;
    attention(out, q, k, v, scores, seq, heads, head_dim);
    free(scores);
    return 0;
}

/* One FLUX.3 block on the CPU: block_forward over x [seq, dim] in place, with
 * the rows in nsegs segments (start, len, mod [3 dim]). w[6]: to_q, to_k,
 * to_v, to_out [dim, dim], ff_in [2 mlp, dim], ff_out [dim, mlp], bf16 as the
 * checkpoints store them. rope tables compact [seq, head_dim / 2]. */
int ref_f3_block(float *x, const uint16_t *const *w, const float *norm_q, const float *norm_k,
                 const int *seg_start, const int *seg_len, const float *const *seg_mod, int nsegs,
                 const float *rope_cos, const float *rope_sin, int seq, int heads, int head_dim, int mlp,
                 float eps) {
    iris_transformer_flux3_t tf;
    f3_block_t b;
    f3_work_t work;
    f3_segment_t segs[8];
    if (nsegs < 1 || nsegs > 8) return -1;
    f3_ctx(&tf, heads, head_dim, 10000.0f);
    tf.mlp = mlp;
    tf.eps = eps;
    if (!ensure_work(&tf, seq, &work)) return -1;
    memset(&b, 0, sizeof(b));
    b.to_q = w[0]; b.to_k = w[1]; b.to_v = w[2]; b.to_out = w[3]; b.ff_in = w[4]; b.ff_out = w[5];
    b.norm_q = norm_q; b.norm_k = norm_k;
    for (int i = 0; i < nsegs; i++) segs[i] = (f3_segment_t){seg_start[i], seg_len[i], seg_mod[i]};
    block_forward(&tf, &b, x, seq, segs, nsegs, rope_cos, rope_sin, &work);
    free(tf.work);
    free(tf.wbuf);
    return 0;
}
