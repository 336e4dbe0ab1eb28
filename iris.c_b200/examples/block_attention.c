/*
 * One transformer block's attention on the device path, written in plain C
 * against include/iris_dev.h exactly as the reference's block code is
 * (forward_dev_flux, iris_transformer_flux.c:3796-3804 and :3834-3839):
 * Q and K go through iris_dev_head_norm_rope in place, then
 * iris_dev_attention runs on the column slices of the fused QKV activation.
 *
 *   block_attention <in.bin> <out.bin>
 *
 * in.bin:  int32 seq, heads; float eps; then qkv bf16 [seq, 3*heads*128],
 *          cos fp32 [seq, 64], sin fp32 [seq, 64], norm_q fp32 [128],
 *          norm_k fp32 [128]
 * out.bin: bf16 [seq, heads*128]
 *
 * Exit codes: 0 done, 2 no usable device, 1 anything else.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "iris_dev.h"

static void *read_block(FILE *f, size_t bytes) {
    void *p = malloc(bytes ? bytes : 1);
    if (!p || fread(p, 1, bytes, f) != bytes) {
        free(p);
        return NULL;
    }
    return p;
}

int main(int argc, char **argv) {
    if (argc != 3) {
        fprintf(stderr, "usage: %s in.bin out.bin\n", argv[0]);
        return 1;
    }
    FILE *f = fopen(argv[1], "rb");
    int32_t hdr[2];
    float eps;
    if (!f || fread(hdr, 4, 2, f) != 2 || fread(&eps, 4, 1, f) != 1) return 1;
    const int seq = hdr[0], heads = hdr[1], hd = 128, dim = heads * hd;
    const size_t qkv_bytes = (size_t)seq * 3 * dim * 2, tab_bytes = (size_t)seq * 64 * 4;
    uint16_t *h_qkv = read_block(f, qkv_bytes);
    float *h_cos = read_block(f, tab_bytes), *h_sin = read_block(f, tab_bytes);
    float *h_wq = read_block(f, hd * 4), *h_wk = read_block(f, hd * 4);
    fclose(f);
    if (!h_qkv || !h_cos || !h_sin || !h_wq || !h_wk) return 1;

    if (!iris_dev_init()) {
        fprintf(stderr, "no usable device\n");
        return 2;
    }
    uint16_t *qkv = iris_dev_alloc(qkv_bytes);
    uint16_t *out = iris_dev_alloc((size_t)seq * dim * 2);
    float *cosd = iris_dev_alloc(tab_bytes), *sind = iris_dev_alloc(tab_bytes);
    float *wq = iris_dev_alloc(hd * 4), *wk = iris_dev_alloc(hd * 4);
    if (!qkv || !out || !cosd || !sind || !wq || !wk) return 1;
    iris_dev_upload(qkv, h_qkv, qkv_bytes);
    iris_dev_upload(cosd, h_cos, tab_bytes);
    iris_dev_upload(sind, h_sin, tab_bytes);
    iris_dev_upload(wq, h_wq, hd * 4);
    iris_dev_upload(wk, h_wk, hd * 4);

    iris_dev_head_norm_rope(qkv, 3 * dim, wq, cosd, sind, seq, heads, hd, eps, 0);
    iris_dev_head_norm_rope(qkv + dim, 3 * dim, wk, cosd, sind, seq, heads, hd, eps, 0);
    iris_dev_attention(out, dim, qkv, qkv + dim, qkv + 2 * dim, 3 * dim, seq, seq, heads, heads, hd,
                       1.0f / sqrtf((float)hd), 0, NULL);

    uint16_t *h_out = malloc((size_t)seq * dim * 2);
    if (!h_out) return 1;
    iris_dev_download(h_out, out, (size_t)seq * dim * 2);
    iris_dev_sync();
    f = fopen(argv[2], "wb");
    if (!f || fwrite(h_out, 2, (size_t)seq * dim, f) != (size_t)seq * dim) return 1;
    fclose(f);
    iris_dev_free(qkv); iris_dev_free(out); iris_dev_free(cosd); iris_dev_free(sind);
    iris_dev_free(wq); iris_dev_free(wk);
    free(h_qkv); free(h_cos); free(h_sin); free(h_wq); free(h_wk); free(h_out);
    printf("block_attention: %s, seq %d, heads %d\n", iris_dev_name(), seq, heads);
    return 0;
}
