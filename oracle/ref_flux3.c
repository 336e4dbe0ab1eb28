/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * Exported wrappers around the `static` FLUX.3 prologue / attention helpers
 * of the reference, compiled from where the reference lies (Makefile REF).
 *
 * Reference functions reached (iris_transformer_flux3.c):
 *   head_rms_norm :172, apply_rope :185, attention :204, rope_rows :282,
 *   image_positions :300, joint_rope :314.
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
