/*
 * TEST INFRASTRUCTURE, not product code: CPU restatement of the reference's
 * joint-attention path. See iris_oracle.h for what pins it.
 *
 * Every function names the reference lines whose arithmetic it follows
 * (paths are those of the reference project).
 */
#include "iris_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------------------
 * Seeded inputs: xoshiro256** seeded through SplitMix64, uniform from the
 * top 53 bits, Box-Muller normal (iris_kernels.c:47-104).
 * ------------------------------------------------------------------------ */

static uint64_t g_s[4] = {0x853c49e6748fea9bULL, 0xda3e39cb94b95bdbULL,
                          0x647c4677a2884327ULL, 0xc6e7918d2e2969f5ULL};

static inline uint64_t rol64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

static uint64_t next_u64(void) {
    uint64_t r = rol64(g_s[1] * 5, 7) * 9, t = g_s[1] << 17;
    g_s[2] ^= g_s[0];
    g_s[3] ^= g_s[1];
    g_s[1] ^= g_s[2];
    g_s[0] ^= g_s[3];
    g_s[2] ^= t;
    g_s[3] = rol64(g_s[3], 45);
    return r;
}

void orc_rng_seed(uint64_t seed) {
    for (int i = 0; i < 4; i++) {
        seed += 0x9e3779b97f4a7c15ULL;
        uint64_t z = seed;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
        g_s[i] = z ^ (z >> 31);
    }
}

float orc_random_uniform(void) {
    return (float)((double)(next_u64() >> 11) * (1.0 / 9007199254740992.0));
}

float orc_random_normal(void) {
    float u1 = orc_random_uniform(), u2 = orc_random_uniform();
    while (u1 == 0.0f) u1 = orc_random_uniform();
    return sqrtf(-2.0f * logf(u1)) * cosf(2.0f * 3.14159265358979323846f * u2);
}

void orc_randn(float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = orc_random_normal();
}

/* ------------------------------------------------------------------------
 * bf16: truncation after adding 0x7FFF + lsb, no NaN case
 * (iris_cuda.cu:236-245).
 * ------------------------------------------------------------------------ */

uint16_t orc_f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float orc_bf2f(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void orc_f32_to_bf16(uint16_t *dst, const float *src, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_f2bf(src[i]);
}

void orc_bf16_to_f32(float *dst, const uint16_t *src, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_bf2f(src[i]);
}

void orc_round_bf16(float *x, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] = orc_bf2f(orc_f2bf(x[i]));
}

/* ------------------------------------------------------------------------
 * iris_kernels.h surface
 * ------------------------------------------------------------------------ */

/* exp(x) = 2^n * poly5(r), n = round(x / ln2), r = x - n ln2
 * (iris_kernels.h:21-32). */
float orc_fast_expf(float x) {
    if (x < -87.3f) return 0.0f;
    if (x > 88.7f) return 1e38f;
    float n = floorf(x * 1.4426950408889634f + 0.5f);
    float r = x - n * 0.6931471805599453f;
    float p = 0.00833333f;
    p = 0.04166667f + r * p;
    p = 0.16666667f + r * p;
    p = 0.5f + r * p;
    p = 1.0f + r * p;
    p = 1.0f + r * p;
    int32_t bits;
    memcpy(&bits, &p, 4);
    bits += (int32_t)n << 23;
    memcpy(&p, &bits, 4);
    return p;
}

/* Row softmax: subtract the row max, exponentiate, divide by the sum
 * (iris_kernels.c:611-633). */
void orc_softmax(float *x, int rows, int cols) {
    for (int r = 0; r < rows; r++) {
        float *row = x + (size_t)r * cols;
        float m = row[0], sum = 0.0f;
        for (int c = 1; c < cols; c++) m = row[c] > m ? row[c] : m;
        for (int c = 0; c < cols; c++) sum += (row[c] = orc_fast_expf(row[c] - m));
        float inv = 1.0f / sum;
        for (int c = 0; c < cols; c++) row[c] *= inv;
    }
}

/* Naive batched attention over [batch, heads, seq, hd] (iris_kernels.c:656-697). */
void orc_attention(float *out, const float *Q, const float *K, const float *V,
                   int batch, int heads, int seq_q, int seq_k, int head_dim, float scale) {
    float *sc = malloc((size_t)seq_q * seq_k * sizeof(float));
    for (int bh = 0; bh < batch * heads; bh++) {
        const float *q = Q + (size_t)bh * seq_q * head_dim;
        const float *k = K + (size_t)bh * seq_k * head_dim;
        const float *v = V + (size_t)bh * seq_k * head_dim;
        float *o = out + (size_t)bh * seq_q * head_dim;
        for (int i = 0; i < seq_q; i++)
            for (int j = 0; j < seq_k; j++) {
                float dot = 0.0f;
                for (int d = 0; d < head_dim; d++) dot += q[i * head_dim + d] * k[j * head_dim + d];
                sc[(size_t)i * seq_k + j] = dot * scale;
            }
        orc_softmax(sc, seq_q, seq_k);
        for (int i = 0; i < seq_q; i++)
            for (int d = 0; d < head_dim; d++) {
                float acc = 0.0f;
                for (int j = 0; j < seq_k; j++) acc += sc[(size_t)i * seq_k + j] * v[j * head_dim + d];
                o[i * head_dim + d] = acc;
            }
    }
    free(sc);
}

/* Online-softmax attention of one head on strided rows, keys visited in
 * tiles of 64: running max / sum per query, rescale of the accumulator when
 * the max moves, sentinel -1e30 for "nothing seen yet", final division
 * (flash_attention_head_tiled, iris_kernels.c:787-886; the small-sequence
 * branch :722-776 computes the same sums key by key). */
static void flash_head(float *out, const float *Q, const float *K, const float *V,
                       int seq_q, int seq_k, int ld, int head_dim, float scale) {
    enum { KT = 64 };
    float sc[KT];
    for (int i = 0; i < seq_q; i++) {
        const float *q = Q + (size_t)i * ld;
        float *o = out + (size_t)i * ld;
        float m = -1e30f, l = 0.0f;
        for (int d = 0; d < head_dim; d++) o[d] = 0.0f;
        for (int k0 = 0; k0 < seq_k; k0 += KT) {
            int kn = seq_k - k0 < KT ? seq_k - k0 : KT;
            float tmax = -1e30f;
            for (int j = 0; j < kn; j++) {
                const float *kr = K + (size_t)(k0 + j) * ld;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; d++) dot += q[d] * kr[d];
                sc[j] = dot * scale;
                if (sc[j] > tmax) tmax = sc[j];
            }
            float nm = tmax > m ? tmax : m;
            if (m > -1e29f) {
                float c = orc_fast_expf(m - nm);
                l *= c;
                for (int d = 0; d < head_dim; d++) o[d] *= c;
            }
            for (int j = 0; j < kn; j++) {
                float w = orc_fast_expf(sc[j] - nm);
                const float *vr = V + (size_t)(k0 + j) * ld;
                l += w;
                for (int d = 0; d < head_dim; d++) o[d] += w * vr[d];
            }
            m = nm;
        }
        float inv = 1.0f / l;
        for (int d = 0; d < head_dim; d++) o[d] *= inv;
    }
}

/* [seq, heads*hd] layout, one head after the other (iris_kernels.c:899-991). */
void orc_flash_attention(float *out, const float *Q, const float *K, const float *V,
                         int seq_q, int seq_k, int heads, int head_dim, float scale) {
    int ld = heads * head_dim;
    for (int h = 0; h < heads; h++)
        flash_head(out + h * head_dim, Q + h * head_dim, K + h * head_dim, V + h * head_dim,
                   seq_q, seq_k, ld, head_dim, scale);
}

/* Split-half 1-D RoPE on [batch, seq, heads, hd] with interleaved (cos, sin)
 * tables [seq, hd/2, 2] (iris_kernels.c:998-1024). */
void orc_apply_rope(float *x, const float *freqs, int batch, int seq, int heads, int head_dim) {
    int half = head_dim / 2;
    for (int b = 0; b < batch; b++)
        for (int s = 0; s < seq; s++)
            for (int h = 0; h < heads; h++) {
                float *v = x + (((size_t)b * seq + s) * heads + h) * head_dim;
                for (int d = 0; d < half; d++) {
                    float c = freqs[((size_t)s * half + d) * 2], sn = freqs[((size_t)s * half + d) * 2 + 1];
                    float a = v[d], bb = v[d + half];
                    v[d] = a * c - bb * sn;
                    v[d + half] = a * sn + bb * c;
                }
            }
}

/* freq_d = theta^(-2d/dim), angle = pos * freq (iris_kernels.c:1026-1038). */
void orc_compute_rope_freqs(float *freqs, const int *pos, int seq, int dim, float theta) {
    int half = dim / 2;
    for (int s = 0; s < seq; s++)
        for (int d = 0; d < half; d++) {
            float f = 1.0f / powf(theta, (float)(2 * d) / (float)dim);
            float a = (float)pos[s] * f;
            freqs[((size_t)s * half + d) * 2] = cosf(a);
            freqs[((size_t)s * half + d) * 2 + 1] = sinf(a);
        }
}

/* ------------------------------------------------------------------------
 * iris_dev.h surface
 * ------------------------------------------------------------------------ */

static void norm_rope_head(float *v, const float *w, const float *c, const float *sn,
                           int head_dim, float eps, int split_half) {
    int half = head_dim / 2;
    float ss = 0.0f;
    for (int d = 0; d < head_dim; d++) ss += v[d] * v[d];
    float inv = 1.0f / sqrtf(ss / head_dim + eps);
    for (int i = 0; i < half; i++) {
        int i0 = split_half ? i : 2 * i, i1 = split_half ? i + half : 2 * i + 1;
        float a = v[i0] * inv * w[i0], b = v[i1] * inv * w[i1];
        v[i0] = a * c[i] - b * sn[i];
        v[i1] = b * c[i] + a * sn[i];
    }
}

void orc_head_norm_rope_f32(float *x, int ld, const float *w,
                            const float *rope_cos, const float *rope_sin,
                            int seq, int heads, int head_dim, float eps, int split_half) {
    int half = head_dim / 2;
    for (int s = 0; s < seq; s++)
        for (int h = 0; h < heads; h++)
            norm_rope_head(x + (size_t)s * ld + (size_t)h * head_dim, w,
                           rope_cos + (size_t)s * half, rope_sin + (size_t)s * half,
                           head_dim, eps, split_half);
}

void orc_head_norm_rope_bf16(uint16_t *x, int ld, const float *w,
                             const float *rope_cos, const float *rope_sin,
                             int seq, int heads, int head_dim, float eps, int split_half) {
    int half = head_dim / 2;
    float *tmp = malloc((size_t)head_dim * sizeof(float));
    for (int s = 0; s < seq; s++)
        for (int h = 0; h < heads; h++) {
            uint16_t *v = x + (size_t)s * ld + (size_t)h * head_dim;
            orc_bf16_to_f32(tmp, v, head_dim);
            norm_rope_head(tmp, w, rope_cos + (size_t)s * half, rope_sin + (size_t)s * half,
                           head_dim, eps, split_half);
            orc_f32_to_bf16(v, tmp, head_dim);
        }
    free(tmp);
}

typedef struct {
    float *out;
    int ldo;
    const float *q, *k, *v;
    int ldi, seq_q, seq_k, heads, kv_heads, head_dim;
    float scale;
    int causal;
    const int *key_mask, *rows;
    int nrows, h0, h1;
} attn_job_t;

/* One full score row per query: scale * q.k over the valid keys, softmax
 * with orc_fast_expf, weighted sum of V. Valid key j: j < causal limit and
 * key_mask[j] != 0 (k_softmax, iris_cuda.cu:514-536); no valid key -> 0. */
static void *attn_worker(void *arg) {
    attn_job_t *w = arg;
    int hd = w->head_dim, group = w->heads / w->kv_heads;
    int nq = w->rows ? w->nrows : w->seq_q;
    float *p = malloc((size_t)w->seq_k * sizeof(float));
    for (int h = w->h0; h < w->h1; h++) {
        int kvh = h / group;
        for (int r = 0; r < nq; r++) {
            int i = w->rows ? w->rows[r] : r;
            const float *q = w->q + (size_t)i * w->ldi + (size_t)h * hd;
            float *o = w->out + (size_t)i * w->ldo + (size_t)h * hd;
            int limit = w->causal ? (i + 1 < w->seq_k ? i + 1 : w->seq_k) : w->seq_k;
            float m = -INFINITY;
            for (int j = 0; j < limit; j++) {
                if (w->key_mask && !w->key_mask[j]) continue;
                const float *kr = w->k + (size_t)j * w->ldi + (size_t)kvh * hd;
                float dot = 0.0f;
                for (int d = 0; d < hd; d++) dot += q[d] * kr[d];
                p[j] = dot * w->scale;
                if (p[j] > m) m = p[j];
            }
            for (int d = 0; d < hd; d++) o[d] = 0.0f;
            if (m == -INFINITY) continue;
            float sum = 0.0f;
            for (int j = 0; j < limit; j++) {
                if (w->key_mask && !w->key_mask[j]) continue;
                float e = orc_fast_expf(p[j] - m);
                const float *vr = w->v + (size_t)j * w->ldi + (size_t)kvh * hd;
                sum += e;
                for (int d = 0; d < hd; d++) o[d] += e * vr[d];
            }
            float inv = 1.0f / sum;
            for (int d = 0; d < hd; d++) o[d] *= inv;
        }
    }
    free(p);
    return NULL;
}

void orc_dev_attention(float *out, int ldo, const float *q, const float *k, const float *v,
                       int ldi, int seq_q, int seq_k, int heads, int kv_heads, int head_dim,
                       float scale, int causal, const int *key_mask,
                       const int *rows, int nrows, int nthreads) {
    if (nthreads <= 0) nthreads = (int)sysconf(_SC_NPROCESSORS_ONLN);
    if (nthreads > heads) nthreads = heads;
    if (nthreads < 1) nthreads = 1;
    pthread_t th[nthreads];
    attn_job_t job[nthreads];
    int started[nthreads];
    for (int t = 0; t < nthreads; t++) {
        job[t] = (attn_job_t){out, ldo, q, k, v, ldi, seq_q, seq_k, heads, kv_heads, head_dim,
                              scale, causal, key_mask, rows, nrows,
                              (int)((long)heads * t / nthreads), (int)((long)heads * (t + 1) / nthreads)};
        started[t] = nthreads > 1 && pthread_create(&th[t], NULL, attn_worker, &job[t]) == 0;
        if (!started[t]) attn_worker(&job[t]);
    }
    for (int t = 0; t < nthreads; t++)
        if (started[t]) pthread_join(th[t], NULL);
}

/* ------------------------------------------------------------------------
 * RoPE tables, compact [seq, hd/2] (one cos / sin per rotated pair)
 * ------------------------------------------------------------------------ */

static void flux_axis(float *c, float *s, int n, float pos, int axis_dim, float theta) {
    for (int d = 0; d < n; d++) {
        float f = 1.0f / powf(theta, (float)(2 * d) / (float)axis_dim);
        float a = pos * f;
        c[d] = cosf(a);
        s[d] = sinf(a);
    }
}

/* Text token i sits at (T, H, W, L) = (0, 0, 0, i): only the L axis turns
 * (compute_rope_text, iris_transformer_flux.c:981-1013). */
void orc_flux_rope_text(float *cos_out, float *sin_out, int txt_seq, int axis_dim, float theta) {
    int ha = axis_dim / 2, half = 4 * ha;
    for (int i = 0; i < txt_seq; i++) {
        float *c = cos_out + (size_t)i * half, *s = sin_out + (size_t)i * half;
        for (int d = 0; d < 3 * ha; d++) { c[d] = 1.0f; s[d] = 0.0f; }
        flux_axis(c + 3 * ha, s + 3 * ha, ha, (float)i, axis_dim, theta);
    }
}

/* Image token (y, x) sits at (t_offset, y, x, 0); t_offset = 0 for the
 * target image, 10 * (i + 1) for reference image i (compute_rope_2d :823,
 * compute_rope_2d_with_t_offset :887, iris.c:1911). */
void orc_flux_rope_image(float *cos_out, float *sin_out, int ph, int pw, int axis_dim,
                         float theta, int t_offset) {
    int ha = axis_dim / 2, half = 4 * ha;
    for (int y = 0; y < ph; y++)
        for (int x = 0; x < pw; x++) {
            size_t r = (size_t)y * pw + x;
            float *c = cos_out + r * half, *s = sin_out + r * half;
            if (t_offset == 0) {
                for (int d = 0; d < ha; d++) { c[d] = 1.0f; s[d] = 0.0f; }
            } else {
                flux_axis(c, s, ha, (float)t_offset, axis_dim, theta);
            }
            flux_axis(c + ha, s + ha, ha, (float)y, axis_dim, theta);
            flux_axis(c + 2 * ha, s + 2 * ha, ha, (float)x, axis_dim, theta);
            for (int d = 3 * ha; d < 4 * ha; d++) { c[d] = 1.0f; s[d] = 0.0f; }
        }
}

static void f3_row(float *c, float *s, const float pos[4], int head_dim, float theta) {
    int ad = head_dim / 4, p = 0;
    for (int ax = 0; ax < 4; ax++)
        for (int j = 0; j < ad / 2; j++, p++) {
            double f = 1.0 / pow((double)theta, (double)(2 * j) / ad);
            double a = (double)pos[ax] * f;
            c[p] = (float)cos(a);
            s[p] = (float)sin(a);
        }
}

int orc_f3_joint_rope(float *cos_out, float *sin_out, int txt_seq, int img_h, int img_w,
                      const int *ref_h, const int *ref_w, int num_refs,
                      int head_dim, float theta) {
    int half = head_dim / 2, row = 0;
    for (int i = 0; i < txt_seq; i++, row++) {
        float pos[4] = {0.0f, 0.0f, 0.0f, (float)i};
        f3_row(cos_out + (size_t)row * half, sin_out + (size_t)row * half, pos, head_dim, theta);
    }
    for (int im = -1; im < num_refs; im++) {
        int h = im < 0 ? img_h : ref_h[im], w = im < 0 ? img_w : ref_w[im];
        float l = im < 0 ? 0.0f : -(float)(im + 1);
        for (int r = 0; r < h; r++)
            for (int c = 0; c < w; c++, row++) {
                float pos[4] = {0.0f, 0.5f * r, 0.5f * c, l};
                f3_row(cos_out + (size_t)row * half, sin_out + (size_t)row * half, pos, head_dim, theta);
            }
    }
    return row;
}

void orc_zi_rope(float *cos_out, float *sin_out, const int *pos, int seq, float theta) {
    static const int dims[3] = {32, 48, 48}, lens[3] = {1024, 512, 512};
    int half = 64;
    for (int s = 0; s < seq; s++) {
        int off = 0;
        for (int ax = 0; ax < 3; ax++) {
            int n = dims[ax] / 2, p = pos[s * 3 + ax];
            int valid = p >= 0 && p < lens[ax];
            for (int i = 0; i < n; i++) {
                float f = 1.0f / powf(theta, (float)(2 * i) / (float)dims[ax]);
                float a = (float)p * f;
                cos_out[(size_t)s * half + off + i] = valid ? cosf(a) : 1.0f;
                sin_out[(size_t)s * half + off + i] = valid ? sinf(a) : 0.0f;
            }
            off += n;
        }
    }
}

int orc_zi_positions(int *pos, int *mask, int ht, int wt, int cap_seq) {
    int img_seq = ht * wt;
    int ip = (img_seq + 31) / 32 * 32, cp = (cap_seq + 31) / 32 * 32;
    memset(pos, 0, (size_t)(ip + cp) * 3 * sizeof(int));
    for (int s = 0; s < ip; s++) {
        mask[s] = s < img_seq;
        if (s < img_seq) {
            pos[3 * s] = cp + 1;
            pos[3 * s + 1] = s / wt;
            pos[3 * s + 2] = s % wt;
        }
    }
    for (int s = 0; s < cp; s++) {
        mask[ip + s] = s < cap_seq;
        pos[3 * (ip + s)] = 1 + s;
    }
    return ip + cp;
}

/* ------------------------------------------------------------------------
 * The operators either side of the attention path inside a block, and one
 * FLUX.2 single-stream block in the arithmetic of the reference's device
 * forward (every stored intermediate rounded to bf16 where the device stores
 * bf16).
 * ------------------------------------------------------------------------ */

/* k_layer_norm_mod, iris_cuda.cu:349-370: mean, variance about the mean,
 * n = (x - mean) * inv; n *= 1 + scale; n += shift; bf16. Sums in double here
 * (the device sums in fp32 in tree order: results agree to one bf16 ulp). */
void orc_layer_norm_mod(uint16_t *out, const float *x, const float *shift, const float *scale,
                        int rows, int dim, float eps) {
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * dim;
        double s = 0;
        for (int i = 0; i < dim; i++) s += xr[i];
        float mean = (float)(s / dim);
        double v = 0;
        for (int i = 0; i < dim; i++) {
            float d = xr[i] - mean;
            v += (double)d * d;
        }
        float inv = 1.0f / sqrtf((float)(v / dim) + eps);
        for (int i = 0; i < dim; i++) {
            float n = (xr[i] - mean) * inv;
            if (scale) n *= 1.0f + scale[i];
            if (shift) n += shift[i];
            out[(size_t)r * dim + i] = orc_f2bf(n);
        }
    }
}

/* k_swiglu, iris_cuda.cu:300-307. */
void orc_swiglu(uint16_t *out, int ldo, const uint16_t *gate, const uint16_t *up, int ldi,
                int rows, int cols) {
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) {
            float g = orc_bf2f(gate[(size_t)r * ldi + c]);
            out[(size_t)r * ldo + c] = orc_f2bf(g / (1.0f + expf(-g)) * orc_bf2f(up[(size_t)r * ldi + c]));
        }
}

/* k_residual, iris_cuda.cu:309-314. */
void orc_residual(float *x, const float *a, const float *gate, int rows, int dim) {
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < dim; c++)
            x[(size_t)r * dim + c] += (gate ? gate[c] : 1.0f) * a[(size_t)r * dim + c];
}

typedef struct {
    float *y;
    int ldy;
    const uint16_t *x;
    int ldx;
    const uint16_t *W;
    int ldw, in, out, r0, r1;
} lin_job_t;

static void *lin_worker(void *arg) {
    lin_job_t *w = arg;
    float *xf = malloc((size_t)w->in * sizeof(float));
    float *wf = malloc((size_t)w->in * sizeof(float));
    for (int c = 0; c < w->out; c++) {
        orc_bf16_to_f32(wf, w->W + (size_t)c * w->ldw, w->in);
        for (int r = w->r0; r < w->r1; r++) {
            orc_bf16_to_f32(xf, w->x + (size_t)r * w->ldx, w->in);
            float acc[8] = {0};
            int i = 0;
            for (; i + 8 <= w->in; i += 8)
                for (int l = 0; l < 8; l++) acc[l] += xf[i + l] * wf[i + l];
            for (; i < w->in; i++) acc[0] += xf[i] * wf[i];
            w->y[(size_t)r * w->ldy + c] =
                ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
        }
    }
    free(xf);
    free(wf);
    return NULL;
}

/* y [rows, out] (fp32, row stride ldy) = x [rows, in] . W [out, in]^T with
 * bf16 operands and fp32 accumulation: the product iris_dev_linear_f32
 * computes (iris_cuda.cu:560-584); rounding y to bf16 afterwards gives
 * iris_dev_linear_bf16 (:463-506). Rows are split over threads. */
void orc_linear(float *y, int ldy, const uint16_t *x, int ldx, const uint16_t *W, int ldw,
                int rows, int in, int out, int nthreads) {
    if (nthreads <= 0) nthreads = (int)sysconf(_SC_NPROCESSORS_ONLN);
    if (nthreads > rows) nthreads = rows;
    if (nthreads < 1) nthreads = 1;
    pthread_t th[nthreads];
    lin_job_t job[nthreads];
    int started[nthreads];
    for (int t = 0; t < nthreads; t++) {
        job[t] = (lin_job_t){y, ldy, x, ldx, W, ldw, in, out,
                             (int)((long)rows * t / nthreads), (int)((long)rows * (t + 1) / nthreads)};
        started[t] = nthreads > 1 && pthread_create(&th[t], NULL, lin_worker, &job[t]) == 0;
        if (!started[t]) lin_worker(&job[t]);
    }
    for (int t = 0; t < nthreads; t++)
        if (started[t]) pthread_join(th[t], NULL);
}

/* One single-stream block as the reference's device forwards issue it
 * (FLUX.2: iris_transformer_flux.c:3828-3845; FLUX.3, rows in segments with
 * their own modulation: iris_transformer_flux3.c:680-703): layer_norm_mod per
 * segment -> linear_bf16 -> head_norm_rope on Q and K -> attention -> swiglu ->
 * linear_f32 -> residual per segment. x [seq, dim] fp32 in place; seg_mod[i] =
 * shift | scale | gate of segment i. Returns 0, or -1 when memory runs out. */
int orc_single_block_segments(float *x, const uint16_t *w_in, const uint16_t *w_out,
                              const float *norm_q, const float *norm_k,
                              const int *seg_start, const int *seg_len, const float *const *seg_mod, int nsegs,
                              const float *rope_cos, const float *rope_sin,
                              int seq, int dim, int heads, int mlp, float eps, const int *key_mask, int nthreads) {
    int hd = dim / heads, ldh = 3 * dim + 2 * mlp, ldc = dim + mlp;
    size_t nh = (size_t)seq * ldh, nc = (size_t)seq * ldc, nd = (size_t)seq * dim;
    uint16_t *norm = malloc(nd * 2), *h = malloc(nh * 2), *cat = malloc(nc * 2);
    float *hf = malloc(nh * sizeof(float)), *qkv = malloc(3 * nd * sizeof(float));
    float *att = malloc(nd * sizeof(float)), *proj = malloc(nd * sizeof(float));
    int rc = -1;
    if (norm && h && cat && hf && qkv && att && proj) {
        for (int g = 0; g < nsegs; g++) {
            size_t off = (size_t)seg_start[g] * dim;
            orc_layer_norm_mod(norm + off, x + off, seg_mod[g], seg_mod[g] + dim, seg_len[g], dim, eps);
        }
        orc_linear(hf, ldh, norm, dim, w_in, dim, seq, dim, ldh, nthreads);
        orc_f32_to_bf16(h, hf, nh);
        orc_head_norm_rope_bf16(h, ldh, norm_q, rope_cos, rope_sin, seq, heads, hd, eps, 0);
        orc_head_norm_rope_bf16(h + dim, ldh, norm_k, rope_cos, rope_sin, seq, heads, hd, eps, 0);
        for (int s = 0; s < seq; s++)
            orc_bf16_to_f32(qkv + (size_t)s * 3 * dim, h + (size_t)s * ldh, 3 * (size_t)dim);
        orc_dev_attention(att, dim, qkv, qkv + dim, qkv + 2 * dim, 3 * dim, seq, seq, heads, heads, hd,
                          1.0f / sqrtf((float)hd), 0, key_mask, NULL, 0, nthreads);
        for (int s = 0; s < seq; s++)
            orc_f32_to_bf16(cat + (size_t)s * ldc, att + (size_t)s * dim, dim);
        orc_swiglu(cat + dim, ldc, h + 3 * dim, h + 3 * dim + mlp, ldh, seq, mlp);
        orc_linear(proj, dim, cat, ldc, w_out, ldc, seq, ldc, dim, nthreads);
        for (int g = 0; g < nsegs; g++) {
            size_t off = (size_t)seg_start[g] * dim;
            orc_residual(x + off, proj + off, seg_mod[g] + 2 * dim, seg_len[g], dim);
        }
        rc = 0;
    }
    free(norm); free(h); free(cat); free(hf); free(qkv); free(att); free(proj);
    return rc;
}

int orc_single_block(float *x, const uint16_t *w_in, const uint16_t *w_out,
                     const float *norm_q, const float *norm_k, const float *mod,
                     const float *rope_cos, const float *rope_sin,
                     int seq, int dim, int heads, int mlp, const int *key_mask, int nthreads) {
    int start = 0;
    return orc_single_block_segments(x, w_in, w_out, norm_q, norm_k, &start, &seq, &mod, 1, rope_cos, rope_sin,
                                     seq, dim, heads, mlp, 1e-6f, key_mask, nthreads);
}

/* One double-stream block as the reference's device forward issues it
 * (iris_transformer_flux.c:3781-3823). x [seq, dim] = [text rows | image
 * rows], in place. w[0] text, w[1] image. */
int orc_double_block(float *x, const orc_stream_weights *txt, const orc_stream_weights *img,
                     const float *rope_cos, const float *rope_sin,
                     int seq, int txt_seq, int dim, int heads, int mlp, const int *key_mask, int nthreads) {
    const orc_stream_weights *w[2] = {txt, img};
    int hd = dim / heads, half = hd / 2;
    int first[2] = {0, txt_seq}, rows[2] = {txt_seq, seq - txt_seq};
    size_t nd = (size_t)seq * dim, nm = (size_t)seq * mlp;
    uint16_t *norm = malloc(nd * 2), *h = malloc(3 * nd * 2), *cat = malloc(nd * 2);
    uint16_t *ff = malloc(2 * nm * 2), *act = malloc(nm * 2);
    float *hf = malloc((3 * nd > 2 * nm ? 3 * nd : 2 * nm) * sizeof(float));
    float *att = malloc(nd * sizeof(float)), *proj = malloc(nd * sizeof(float));
    int rc = -1;
    if (norm && h && cat && ff && act && hf && att && proj) {
        for (int m = 0; m < 2; m++) {
            size_t r0 = (size_t)first[m];
            int n = rows[m];
            uint16_t *qkv = h + 3 * r0 * dim;
            orc_layer_norm_mod(norm, x + r0 * dim, w[m]->mod, w[m]->mod + dim, n, dim, 1e-6f);
            orc_linear(hf, 3 * dim, norm, dim, w[m]->qkv, dim, n, dim, 3 * dim, nthreads);
            orc_f32_to_bf16(qkv, hf, (size_t)n * 3 * dim);
            orc_head_norm_rope_bf16(qkv, 3 * dim, w[m]->norm_q, rope_cos + r0 * half, rope_sin + r0 * half,
                                    n, heads, hd, 1e-6f, 0);
            orc_head_norm_rope_bf16(qkv + dim, 3 * dim, w[m]->norm_k, rope_cos + r0 * half, rope_sin + r0 * half,
                                    n, heads, hd, 1e-6f, 0);
        }
        orc_bf16_to_f32(hf, h, 3 * nd);
        orc_dev_attention(att, dim, hf, hf + dim, hf + 2 * dim, 3 * dim, seq, seq, heads, heads, hd,
                          1.0f / sqrtf((float)hd), 0, key_mask, NULL, 0, nthreads);
        orc_f32_to_bf16(cat, att, nd);
        for (int m = 0; m < 2; m++) {
            size_t r0 = (size_t)first[m];
            orc_linear(proj, dim, cat + r0 * dim, dim, w[m]->proj, dim, rows[m], dim, dim, nthreads);
            orc_residual(x + r0 * dim, proj, w[m]->mod + 2 * dim, rows[m], dim);
        }
        for (int m = 0; m < 2; m++) {
            size_t r0 = (size_t)first[m];
            int n = rows[m];
            orc_layer_norm_mod(norm, x + r0 * dim, w[m]->mod + 3 * dim, w[m]->mod + 4 * dim, n, dim, 1e-6f);
            orc_linear(hf, 2 * mlp, norm, dim, w[m]->ff_in, dim, n, dim, 2 * mlp, nthreads);
            orc_f32_to_bf16(ff, hf, (size_t)n * 2 * mlp);
            orc_swiglu(act, mlp, ff, ff + mlp, 2 * mlp, n, mlp);
            orc_linear(proj, dim, act, mlp, w[m]->ff_out, mlp, n, mlp, dim, nthreads);
            orc_residual(x + r0 * dim, proj, w[m]->mod + 5 * dim, n, dim);
        }
        rc = 0;
    }
    free(norm); free(h); free(cat); free(ff); free(act); free(hf); free(att); free(proj);
    return rc;
}

/* k_rms_norm, iris_cuda.cu:372-386: out = x * inv * w, times (1 + scale) when
 * scale is given; sum of squares in double here. */
void orc_rms_norm_mod(uint16_t *out, const float *x, const float *w, const float *scale,
                      int rows, int dim, float eps) {
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * dim;
        double s = 0;
        for (int i = 0; i < dim; i++) s += (double)xr[i] * xr[i];
        float inv = 1.0f / sqrtf((float)(s / dim) + eps);
        for (int i = 0; i < dim; i++) {
            float v = xr[i] * inv * w[i];
            if (scale) v *= 1.0f + scale[i];
            out[(size_t)r * dim + i] = orc_f2bf(v);
        }
    }
}

/* k_rms_norm_residual, iris_cuda.cu:388-400: x += tanh(gate) * a * inv * w. */
void orc_rms_norm_residual(float *x, const float *a, const float *w, const float *gate,
                           int rows, int dim, float eps) {
    for (int r = 0; r < rows; r++) {
        const float *ar = a + (size_t)r * dim;
        double s = 0;
        for (int i = 0; i < dim; i++) s += (double)ar[i] * ar[i];
        float inv = 1.0f / sqrtf((float)(s / dim) + eps);
        for (int i = 0; i < dim; i++)
            x[(size_t)r * dim + i] += (gate ? tanhf(gate[i]) : 1.0f) * (ar[i] * inv * w[i]);
    }
}

/* One Z-Image block as zi_dev_block issues it
 * (iris_transformer_zimage.c:1940-1959), in place on x [seq, dim]. mod [4 dim]
 * = scale_msa | gate_msa | scale_mlp | gate_mlp or NULL. */
int orc_zimage_block(float *x, const orc_zimage_weights *w, const float *mod,
                     const float *rope_cos, const float *rope_sin,
                     int seq, int dim, int heads, int ff, const int *key_mask, int nthreads) {
    int hd = dim / heads;
    float eps = 1e-5f;
    size_t nd = (size_t)seq * dim, nf = (size_t)seq * ff;
    uint16_t *norm = malloc(nd * 2), *h = malloc(3 * nd * 2), *act = malloc((nd > nf ? nd : nf) * 2);
    uint16_t *ffh = malloc(2 * nf * 2);
    float *hf = malloc((3 * nd > 2 * nf ? 3 * nd : 2 * nf) * sizeof(float));
    float *att = malloc(nd * sizeof(float)), *out = malloc(nd * sizeof(float));
    int rc = -1;
    if (norm && h && act && ffh && hf && att && out) {
        orc_rms_norm_mod(norm, x, w->attn_norm1, mod, seq, dim, eps);
        orc_linear(hf, 3 * dim, norm, dim, w->qkv, dim, seq, dim, 3 * dim, nthreads);
        orc_f32_to_bf16(h, hf, 3 * nd);
        orc_head_norm_rope_bf16(h, 3 * dim, w->norm_q, rope_cos, rope_sin, seq, heads, hd, eps, 0);
        orc_head_norm_rope_bf16(h + dim, 3 * dim, w->norm_k, rope_cos, rope_sin, seq, heads, hd, eps, 0);
        orc_bf16_to_f32(hf, h, 3 * nd);
        orc_dev_attention(att, dim, hf, hf + dim, hf + 2 * dim, 3 * dim, seq, seq, heads, heads, hd,
                          1.0f / sqrtf((float)hd), 0, key_mask, NULL, 0, nthreads);
        orc_f32_to_bf16(act, att, nd);
        orc_linear(out, dim, act, dim, w->proj, dim, seq, dim, dim, nthreads);
        orc_rms_norm_residual(x, out, w->attn_norm2, mod ? mod + dim : NULL, seq, dim, eps);
        orc_rms_norm_mod(norm, x, w->ffn_norm1, mod ? mod + 2 * dim : NULL, seq, dim, eps);
        orc_linear(hf, 2 * ff, norm, dim, w->ff_in, dim, seq, dim, 2 * ff, nthreads);
        orc_f32_to_bf16(ffh, hf, 2 * nf);
        orc_swiglu(act, ff, ffh, ffh + ff, 2 * ff, seq, ff);
        orc_linear(out, dim, act, ff, w->ff_out, ff, seq, ff, dim, nthreads);
        orc_rms_norm_residual(x, out, w->ffn_norm2, mod ? mod + 3 * dim : NULL, seq, dim, eps);
        rc = 0;
    }
    free(norm); free(h); free(act); free(ffh); free(hf); free(att); free(out);
    return rc;
}

/* ------------------------------------------------------------------------
 * Metrics
 * ------------------------------------------------------------------------ */

void orc_compare_heads(const float *a, int lda, const float *b, int ldb, int seq, int heads,
                       int head_dim, const int *rows, int nrows,
                       float *max_abs, float *cosine) {
    int n = rows ? nrows : seq;
    for (int h = 0; h < heads; h++) {
        double dot = 0, na = 0, nb = 0;
        float mx = 0.0f;
        for (int r = 0; r < n; r++) {
            int i = rows ? rows[r] : r;
            const float *pa = a + (size_t)i * lda + (size_t)h * head_dim;
            const float *pb = b + (size_t)i * ldb + (size_t)h * head_dim;
            for (int d = 0; d < head_dim; d++) {
                float diff = fabsf(pa[d] - pb[d]);
                if (mx == mx && (diff > mx || diff != diff)) mx = diff;   /* NaN sticks */
                dot += (double)pa[d] * pb[d];
                na += (double)pa[d] * pa[d];
                nb += (double)pb[d] * pb[d];
            }
        }
        max_abs[h] = mx;
        cosine[h] = (na > 0 && nb > 0) ? (float)(dot / sqrt(na * nb)) : (na == nb ? 1.0f : 0.0f);
    }
}
