/*
 * Host-pointer fp32 surface (iris_kernels.h): the attention, softmax and
 * RoPE entry points of the reference's CPU kernel file, executed on the GPU.
 * Each call uploads its operands into library scratch, runs the device
 * kernels and downloads the result before returning, so it behaves like the
 * synchronous CPU functions it replaces (iris_kernels.c:611-1038).
 */
#include "common.cuh"

#include <math.h>

#include "iris_dev.h"
#include "iris_kernels.h"
#include "kernels.h"

namespace iris_b200 {

/* f32 [b, h, s, d] -> bf16 [b][s, h*d] (to_shd) or bf16 [b][s, h*d] -> f32
 * [b, h, s, d]; with b = h_outer = 1 it is a plain cast. */
__global__ void k_bhsd_to_bf16(uint16_t *dst, const float *src, int heads, int seq, int hd, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int d = (int)(i % hd);
    size_t r = i / hd;
    int s = (int)(r % seq);
    r /= seq;
    int h = (int)(r % heads);
    size_t b = r / heads;
    dst[((b * seq + s) * heads + h) * hd + d] = f2bf(src[i]);
}

__global__ void k_bf16_to_bhsd(float *dst, const uint16_t *src, int heads, int seq, int hd, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int d = (int)(i % hd);
    size_t r = i / hd;
    int s = (int)(r % seq);
    r /= seq;
    int h = (int)(r % heads);
    size_t b = r / heads;
    dst[i] = bf2f(src[((b * seq + s) * heads + h) * hd + d]);
}

__global__ void k_bf16_to_f32(float *dst, const uint16_t *src, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = bf2f(src[i]);
}

/* One block per row: max, exp, sum, scale (iris_kernels.c:611-633). */
__global__ void k_softmax_rows(float *x, int cols) {
    __shared__ float red[32];
    float *row = x + (size_t)blockIdx.x * cols;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, row[c]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nw; w++) m = fmaxf(m, red[w]);
    __syncthreads();
    float sum = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float e = expf(row[c] - m);
        row[c] = e;
        sum += e;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.0f;
    for (int w = 0; w < nw; w++) sum += red[w];
    float inv = 1.0f / sum;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] *= inv;
}

/* Split-half rotation of x[b, s, h, :] by freqs[s, :, (cos, sin)]
 * (iris_kernels.c:998-1024): one thread per rotated pair. */
__global__ void k_apply_rope(float *x, const float *freqs, int seq, int heads, int hd, size_t npairs) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    int half = hd / 2;
    int d = (int)(i % half);
    size_t vec = i / half;                       /* (b * seq + s) * heads + h */
    int s = (int)((vec / heads) % seq);
    float c = freqs[((size_t)s * half + d) * 2], sn = freqs[((size_t)s * half + d) * 2 + 1];
    float *v = x + vec * hd;
    float a = v[d], b = v[d + half];
    v[d] = a * c - b * sn;
    v[d + half] = a * sn + b * c;
}

/* (cos, sin)(pos * theta^(-2d/dim)) (iris_kernels.c:1026-1038). */
__global__ void k_rope_freqs(float *freqs, const int *pos, int seq, int dim, float theta) {
    int half = dim / 2;
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= seq * half) return;
    int s = i / half, d = i % half;
    float f = 1.0f / powf(theta, (float)(2 * d) / (float)dim);
    float a = (float)pos[s] * f;
    freqs[(size_t)i * 2] = cosf(a);
    freqs[(size_t)i * 2 + 1] = sinf(a);
}

static unsigned blocks_for(size_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

static size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

/* Attention of `batch` independent problems given in [b, h, s, d] layout
 * (heads_outer = 1 makes it the [s, h*d] layout of the transformers). */
static void host_attention(float *out, const float *Q, const float *K, const float *V, int batch,
                           int heads, int seq_q, int seq_k, int head_dim, float scale, bool bhsd,
                           const char *name) {
    if (!require_device(name)) return;
    if (batch <= 0 || heads <= 0 || seq_q <= 0 || head_dim <= 0) return;
    size_t nq = (size_t)batch * heads * seq_q * head_dim, nk = (size_t)batch * heads * seq_k * head_dim;
    size_t f32_bytes = align256((nq > nk ? nq : nk) * 4);
    size_t bytes = f32_bytes + 2 * align256(nq * 2) + 2 * align256(nk * 2);
    char *base = (char *)ensure_scratch(bytes);
    if (!base) return;
    float *stage = (float *)base;
    uint16_t *q16 = (uint16_t *)(base + f32_bytes);
    uint16_t *k16 = (uint16_t *)((char *)q16 + align256(nq * 2));
    uint16_t *v16 = (uint16_t *)((char *)k16 + align256(nk * 2));
    uint16_t *o16 = (uint16_t *)((char *)v16 + align256(nk * 2));
    int ho = bhsd ? heads : 1;                  /* heads as an outer axis of the host layout */
    int inner = bhsd ? head_dim : heads * head_dim;
    const float *src[3] = {Q, K, V};
    uint16_t *dst[3] = {q16, k16, v16};
    for (int i = 0; i < 3; i++) {
        size_t n = i == 0 ? nq : nk;
        int seq = i == 0 ? seq_q : seq_k;
        if (n == 0) continue;
        iris_dev_upload(stage, src[i], n * 4);
        k_bhsd_to_bf16<<<blocks_for(n, 256), 256, 0, g.stream>>>(dst[i], stage, ho, seq, inner, n);
        if (!after_launch(name)) return;
    }
    int ld = heads * head_dim;
    for (int b = 0; b < batch; b++) {
        int rc = iris_b200_attention_ex(o16 + (size_t)b * seq_q * ld, ld, q16 + (size_t)b * seq_q * ld,
                                        k16 + (size_t)b * seq_k * ld, v16 + (size_t)b * seq_k * ld, ld,
                                        seq_q, seq_k, heads, heads, head_dim, scale, 0, NULL,
                                        IRIS_B200_KERNEL_AUTO);
        if (rc != IRIS_B200_OK) return;
    }
    k_bf16_to_bhsd<<<blocks_for(nq, 256), 256, 0, g.stream>>>(stage, o16, ho, seq_q, inner, nq);
    if (!after_launch(name)) return;
    iris_dev_download(out, stage, nq * 4);
}

}  // namespace iris_b200

using namespace iris_b200;

extern "C" {

void iris_flash_attention(float *out, const float *Q, const float *K, const float *V,
                          int seq_q, int seq_k, int heads, int head_dim, float scale) {
    host_attention(out, Q, K, V, 1, heads, seq_q, seq_k, head_dim, scale, false, "iris_flash_attention");
}

void iris_attention(float *out, const float *Q, const float *K, const float *V,
                    int batch, int heads, int seq_q, int seq_k, int head_dim, float scale) {
    host_attention(out, Q, K, V, batch, heads, seq_q, seq_k, head_dim, scale, true, "iris_attention");
}

void iris_softmax(float *x, int rows, int cols) {
    if (!require_device("iris_softmax") || rows <= 0 || cols <= 0) return;
    size_t bytes = (size_t)rows * cols * 4;
    float *d = (float *)ensure_scratch(bytes);
    if (!d) return;
    iris_dev_upload(d, x, bytes);
    k_softmax_rows<<<rows, 256, 0, g.stream>>>(d, cols);
    if (!after_launch("iris_softmax")) return;
    iris_dev_download(x, d, bytes);
}

/* The reference exports the same routine under a second name that its BLAS
 * attention variants call (iris_kernels.h:159). */
void iris_softmax_cpu(float *x, int rows, int cols) { iris_softmax(x, rows, cols); }

void iris_apply_rope(float *x, const float *freqs, int batch, int seq, int heads, int head_dim) {
    if (!require_device("iris_apply_rope") || batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0) return;
    size_t n = (size_t)batch * seq * heads * head_dim, nf = (size_t)seq * head_dim;
    char *base = (char *)ensure_scratch(align256(n * 4) + nf * 4);
    if (!base) return;
    float *dx = (float *)base, *df = (float *)(base + align256(n * 4));
    iris_dev_upload(dx, x, n * 4);
    iris_dev_upload(df, freqs, nf * 4);
    k_apply_rope<<<blocks_for(n / 2, 256), 256, 0, g.stream>>>(dx, df, seq, heads, head_dim, n / 2);
    if (!after_launch("iris_apply_rope")) return;
    iris_dev_download(x, dx, n * 4);
}

void iris_compute_rope_freqs(float *freqs, const int *pos, int seq, int dim, float theta) {
    if (!require_device("iris_compute_rope_freqs") || seq <= 0 || dim <= 1) return;
    size_t nf = (size_t)seq * (dim / 2) * 2;
    char *base = (char *)ensure_scratch(align256(nf * 4) + (size_t)seq * 4);
    if (!base) return;
    float *df = (float *)base;
    int *dp = (int *)(base + align256(nf * 4));
    iris_dev_upload(dp, pos, (size_t)seq * 4);
    k_rope_freqs<<<blocks_for(nf / 2, 256), 256, 0, g.stream>>>(df, dp, seq, dim, theta);
    if (!after_launch("iris_compute_rope_freqs")) return;
    iris_dev_download(freqs, df, nf * 4);
}

}  // extern "C"
