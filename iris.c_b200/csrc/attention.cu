/*
 * iris_dev_attention: argument checks and kernel choice.
 *
 * The transformer-block domain (head_dim 128, heads == kv_heads, non-causal,
 * aligned views) runs on the tcgen05 kernel; every other combination the
 * reference accepts (GQA, causal, other head sizes, odd alignment:
 * iris_cuda.cu:897-936) runs on the general CUDA-core kernel. There is no
 * CPU path: without a device the call fails.
 */
#include "common.cuh"

#include "iris_dev.h"
#include "kernels.h"

using namespace iris_b200;

namespace iris_b200 {

/* Pointers, counts and row strides every attention entry point insists on:
 * a stride shorter than a row of heads would make rows overlap (inputs) or
 * let the output run past its buffer. out may be NULL where an entry point
 * allows it (ldo is then not looked at). */
int check_attention_args(const char *op, const void *out, const void *q, const void *k, const void *v, int ldo,
                         int ldq, int ldkv, int seq_q, int seq_k, int heads, int kv_heads, int head_dim) {
    if (!q || !k || !v || seq_q < 0 || seq_k < 0 || heads <= 0 || kv_heads <= 0 ||
        heads % kv_heads != 0 || head_dim <= 0 || (out && ldo < heads * head_dim) || ldq < heads * head_dim ||
        ldkv < kv_heads * head_dim) {
        set_error(IRIS_B200_EINVAL, op, "bad argument");
        return IRIS_B200_EINVAL;
    }
    return IRIS_B200_OK;
}

}  // namespace iris_b200

extern "C" int iris_b200_attention_kernel_for(const void *out, int ldo, const void *q, const void *k,
                                              const void *v, int ldi, int heads, int kv_heads,
                                              int head_dim, int causal) {
    return sm100_supported(out, ldo, q, k, v, ldi, heads, kv_heads, head_dim, causal, 1.0f)
               ? IRIS_B200_KERNEL_TCGEN05 : IRIS_B200_KERNEL_GENERIC;
}

extern "C" int iris_b200_attention_ex(uint16_t *out, int ldo,
                                      const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                      int ldi, int seq_q, int seq_k, int heads, int kv_heads,
                                      int head_dim, float scale, int causal,
                                      const int *key_mask, int kernel) {
    if (!require_device("attention")) return IRIS_B200_ENODEV;
    if (!out) {
        set_error(IRIS_B200_EINVAL, "attention", "bad argument");
        return IRIS_B200_EINVAL;
    }
    int rc = check_attention_args("attention", out, q, k, v, ldo, ldi, ldi, seq_q, seq_k, heads, kv_heads, head_dim);
    if (rc != IRIS_B200_OK) return rc;
    if (seq_q == 0) return IRIS_B200_OK;
    bool fast = sm100_supported(out, ldo, q, k, v, ldi, heads, kv_heads, head_dim, causal, scale);
    if (kernel == IRIS_B200_KERNEL_TCGEN05 && !fast) {
        set_error(IRIS_B200_EUNSUPPORTED, "attention", "arguments outside the tcgen05 kernel's domain");
        return IRIS_B200_EUNSUPPORTED;
    }
    if (kernel == IRIS_B200_KERNEL_GENERIC) fast = false;
    if (fast)
        return launch_attention_sm100(attn_args(out, ldo, q, ldi, k, v, ldi, seq_q, seq_k, heads, scale, key_mask));
    return launch_attention_generic(out, ldo, q, k, v, ldi, seq_q, seq_k, heads, kv_heads, head_dim,
                                    scale, causal, key_mask);
}

extern "C" void iris_dev_attention(uint16_t *out, int ldo,
                                   const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                   int ldi, int seq_q, int seq_k, int heads, int kv_heads,
                                   int head_dim, float scale, int causal,
                                   const int *key_mask) {
    iris_b200_attention_ex(out, ldo, q, k, v, ldi, seq_q, seq_k, heads, kv_heads, head_dim, scale,
                           causal, key_mask, IRIS_B200_KERNEL_AUTO);
}
