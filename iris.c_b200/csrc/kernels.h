/* Internal launch functions shared between translation units. */
#pragma once
#include <stdint.h>

namespace iris_b200 {

int launch_attention_generic(uint16_t *out, int ldo, const uint16_t *q, const uint16_t *k,
                             const uint16_t *v, int ldi, int seq_q, int seq_k, int heads,
                             int kv_heads, int head_dim, float scale, int causal,
                             const int *key_mask);

bool sm100_supported(const void *out, int ldo, const void *q, const void *k, const void *v, int ldi,
                     int heads, int kv_heads, int head_dim, int causal, float scale);

int launch_attention_sm100(uint16_t *out, int ldo, const uint16_t *q, int ldq, const uint16_t *k,
                           const uint16_t *v, int ldkv, int seq_q, int seq_k, int heads, float scale,
                           const int *key_mask, int acc_mode, float *o_acc, float *lse_acc,
                           float *debug, const uint32_t *desc_override, int max_split = 2);

void sm100_release(void);

/* Clears the arrival words of the key-split scratch (after a device wait timed out). */
void sm100_reset_split(void);

}  // namespace iris_b200
