/*
 * Prologue of the attention path: per-head RMSNorm, pair rotation (RoPE) and
 * bf16 store, in place on the Q / K column slices of the fused projection
 * output. HBM-bound: every element is read once and written once.
 *
 * Fast kernels (head_dim 128, 16-byte aligned rows): 16 lanes own one
 * (token, head) unit, each lane one 16-byte vector of 8 consecutive bf16.
 * With consecutive pairs (the three transformers) both members of a pair sit
 * in the same lane and a 16-lane group walks all heads of one token, so the
 * token's angles and the weights are folded once into per-lane constants
 * (k_head_norm_rope_128_tok). With split-half pairing lane l exchanges with
 * lane l ^ 8 (k_head_norm_rope_128<true>). The sum of squares is reduced
 * with four shuffles inside the 16-lane group. Several units are in flight
 * per thread so that enough bytes are outstanding to fill the HBM pipe. Q
 * and K of a block go through one launch.
 *
 * Arithmetic follows the reference kernel (iris_cuda.cu:403-420): widen to
 * fp32, inv = rsqrt(mean(x^2) + eps), a = x * (inv * w), rotate, one
 * round-to-nearest-even to bf16.
 */
#include "common.cuh"

#include "iris_dev.h"

namespace iris_b200 {

static constexpr int kUnroll = 2;        /* units in flight per 16-lane group */
static constexpr int kBlocksPerSM = 5;   /* register budget: 65536 / (5 * 256) = 51 */
static constexpr int kThreads = 256;

struct alignas(16) Vec8 {
    uint32_t w[4];
};

template <bool SPLIT_HALF>
__global__ void __launch_bounds__(kThreads, kBlocksPerSM)
k_head_norm_rope_128(uint16_t *__restrict__ q, uint16_t *__restrict__ k, int ld,
                     const float *__restrict__ wq, const float *__restrict__ wk,
                     const float *__restrict__ rope_cos, const float *__restrict__ rope_sin,
                     int seq, int heads, float eps) {
    const int lane16 = threadIdx.x & 15;
    const int group = (int)(((long long)blockIdx.x * kThreads + threadIdx.x) >> 4);
    const int ngroups = (int)(((long long)gridDim.x * kThreads) >> 4);
    const int per_tok = k ? 2 * heads : heads;      /* units of one token: Q heads then K heads */

    /* This lane always owns dims [8 * lane16, 8 * lane16 + 8) of a head; its
     * eight weights are re-read (L1 hits) per unit to keep registers low. */
    /* Pairs whose angle this lane needs: consecutive -> pairs 4l..4l+3;
     * split-half -> pairs 8(l & 7)..+7, shared with lane l ^ 8. */
    const int rope_off = SPLIT_HALF ? (lane16 & 7) * 8 : lane16 * 4;

    /* Units are dealt round-robin to the 16-lane groups; (token, unit in
     * token) advance by a fixed step, so the loop has no division. */
    const int step_tok = ngroups / per_tok, step_hu = ngroups - step_tok * per_tok;
    int tok_next = group / per_tok, hu_next = group - tok_next * per_tok;

    while (tok_next < seq) {
        Vec8 v[kUnroll];
        uint16_t *ptr[kUnroll];
        int tok[kUnroll];
        bool isk[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; i++) {
            bool ok = tok_next < seq;
            int hu = hu_next;
            tok[i] = tok_next;
            isk[i] = hu >= heads;
            int h = isk[i] ? hu - heads : hu;
            ptr[i] = ok ? (isk[i] ? k : q) + (size_t)tok_next * ld + h * 128 + lane16 * 8 : nullptr;
            if (ok) v[i] = *reinterpret_cast<const Vec8 *>(ptr[i]);
            tok_next += step_tok;
            hu_next += step_hu;
            if (hu_next >= per_tok) {
                hu_next -= per_tok;
                tok_next++;
            }
        }
#pragma unroll
        for (int i = 0; i < kUnroll; i++) {
            /* Uniform inside the 16-lane group: all its lanes share the unit. */
            bool ok = ptr[i] != nullptr;
            float x[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                x[2 * j] = ok ? bf_lo(v[i].w[j]) : 0.0f;
                x[2 * j + 1] = ok ? bf_hi(v[i].w[j]) : 0.0f;
            }
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) ss += x[j] * x[j];
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
            {
                const float4 *wp = reinterpret_cast<const float4 *>((isk[i] ? wk : wq) + lane16 * 8);
                float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
                x[0] *= inv * w0.x; x[1] *= inv * w0.y; x[2] *= inv * w0.z; x[3] *= inv * w0.w;
                x[4] *= inv * w1.x; x[5] *= inv * w1.y; x[6] *= inv * w1.z; x[7] *= inv * w1.w;
            }

            if (SPLIT_HALF) {
                float c[8], sn[8];
                if (ok) {
                    const float4 *cp = reinterpret_cast<const float4 *>(rope_cos + (size_t)tok[i] * 64 + rope_off);
                    const float4 *sp = reinterpret_cast<const float4 *>(rope_sin + (size_t)tok[i] * 64 + rope_off);
                    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
                    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w;
                    c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
                    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w;
                    sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
                }
                bool upper = lane16 >= 8;       /* holds the second member of each pair */
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float other = __shfl_xor_sync(0xffffffffu, x[j], 8);
                    if (ok) x[j] = upper ? x[j] * c[j] + other * sn[j] : x[j] * c[j] - other * sn[j];
                }
            } else if (ok) {
                float4 c = *reinterpret_cast<const float4 *>(rope_cos + (size_t)tok[i] * 64 + rope_off);
                float4 s = *reinterpret_cast<const float4 *>(rope_sin + (size_t)tok[i] * 64 + rope_off);
                float cc[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float a = x[2 * j], b = x[2 * j + 1];
                    x[2 * j] = a * cc[j] - b * sn[j];
                    x[2 * j + 1] = b * cc[j] + a * sn[j];
                }
            }
            if (ok) {
                Vec8 o;
#pragma unroll
                for (int j = 0; j < 4; j++) o.w[j] = cvt_bf16x2(x[2 * j], x[2 * j + 1]);
                *reinterpret_cast<Vec8 *>(ptr[i]) = o;
            }
        }
    }
}

/* Consecutive-pair kernel, token-major: a 16-lane group owns one (token,
 * Q | K) row segment and walks its heads. The lane's four (cos, sin) pairs
 * and eight weights are loaded once per token and folded into four products
 * per pair (cos * w, sin * w), so a head costs one 16-byte load, the sum of
 * squares, six FMA-pipe operations per pair and one 16-byte store. kHeadsInFlight
 * heads are loaded before the first is used. */
static constexpr int kHeadsInFlight = 4;
/* Four heads in flight and four blocks per SM is the measured optimum at the
 * Klein-4B shape (115.6 MB: 23.1 us, against 22.7 us for a plain copy kernel
 * that reads and writes the same strided columns): more resident warps (5, 6,
 * 8 blocks) or more heads in flight, or a prefetch of the next heads, were
 * all slower (24 - 48 us). */
static constexpr int kTokBlocksPerSM = 4;

__global__ void __launch_bounds__(kThreads, kTokBlocksPerSM)
k_head_norm_rope_128_tok(uint16_t *__restrict__ q, uint16_t *__restrict__ k, int ld,
                         const float *__restrict__ wq, const float *__restrict__ wk,
                         const float *__restrict__ rope_cos, const float *__restrict__ rope_sin,
                         int seq, int heads, float eps) {
    /* A launch that follows with programmatic stream serialisation (the
     * attention) may set itself up while this grid runs; it waits for this
     * grid's completion before it reads anything. */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane16 = threadIdx.x & 15;
    const int group = (int)(((long long)blockIdx.x * kThreads + threadIdx.x) >> 4);
    const int ngroups = (int)(((long long)gridDim.x * kThreads) >> 4);
    const int nseg = k ? 2 * seq : seq;             /* segment = (token, Q | K) */

    /* Both groups of a warp run the same number of rounds (the shuffles
     * below name the whole warp); a group past the end idles with `live` off. */
    for (int seg0 = group & ~1; seg0 < nseg; seg0 += ngroups) {
        const int seg = seg0 + (group & 1);
        const bool live = seg < nseg;
        const bool isk = live && seg >= seq;
        const int tok = live ? (isk ? seg - seq : seg) : 0;
        uint16_t *base = (isk ? k : q) + (size_t)tok * ld + lane16 * 8;
        const float4 c = *reinterpret_cast<const float4 *>(rope_cos + (size_t)tok * 64 + lane16 * 4);
        const float4 sn = *reinterpret_cast<const float4 *>(rope_sin + (size_t)tok * 64 + lane16 * 4);
        const float4 *wp = reinterpret_cast<const float4 *>((isk ? wk : wq) + lane16 * 8);
        const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
        const float cc[4] = {c.x, c.y, c.z, c.w}, ss4[4] = {sn.x, sn.y, sn.z, sn.w};
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float cw0[4], sw1[4], cw1[4], sw0[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            cw0[j] = cc[j] * ww[2 * j];
            sw1[j] = ss4[j] * ww[2 * j + 1];
            cw1[j] = cc[j] * ww[2 * j + 1];
            sw0[j] = ss4[j] * ww[2 * j];
        }
        for (int h0 = 0; h0 < heads; h0 += kHeadsInFlight) {
            Vec8 v[kHeadsInFlight];
#pragma unroll
            for (int i = 0; i < kHeadsInFlight; i++)
                if (live && h0 + i < heads) v[i] = *reinterpret_cast<const Vec8 *>(base + (h0 + i) * 128);
#pragma unroll
            for (int i = 0; i < kHeadsInFlight; i++) {
                const bool ok = live && h0 + i < heads;
                float x[8];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    x[2 * j] = ok ? bf_lo(v[i].w[j]) : 0.0f;
                    x[2 * j + 1] = ok ? bf_hi(v[i].w[j]) : 0.0f;
                }
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) ss = fmaf(x[j], x[j], ss);
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
                if (ok) {
                    Vec8 o;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float a = x[2 * j], b = x[2 * j + 1];
                        o.w[j] = cvt_bf16x2((a * cw0[j] - b * sw1[j]) * inv, (b * cw1[j] + a * sw0[j]) * inv);
                    }
                    *reinterpret_cast<Vec8 *>(base + (h0 + i) * 128) = o;
                }
            }
        }
    }
}

/* Any even head_dim, any alignment: one warp per (token, head), 2-byte
 * accesses. Covers the argument domains the fast kernel does not. */
__global__ void k_head_norm_rope_any(uint16_t *x, int ld, const float *w,
                                     const float *rope_cos, const float *rope_sin,
                                     int seq, int heads, int head_dim, float eps, int split_half) {
    int lane = threadIdx.x & 31;
    long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    long long units = (long long)seq * heads;
    if (unit >= units) return;
    int s = (int)(unit / heads), h = (int)(unit % heads), half = head_dim / 2;
    uint16_t *v = x + (size_t)s * ld + (size_t)h * head_dim;
    float ss = 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
        float a = bf2f(v[d]);
        ss += a * a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float inv = rsqrtf(ss / head_dim + eps);
    for (int i = lane; i < half; i += 32) {
        int i0 = split_half ? i : 2 * i, i1 = split_half ? i + half : 2 * i + 1;
        float a = bf2f(v[i0]) * (inv * w[i0]), b = bf2f(v[i1]) * (inv * w[i1]);
        float c = rope_cos[(size_t)s * half + i], sn = rope_sin[(size_t)s * half + i];
        v[i0] = f2bf(a * c - b * sn);
        v[i1] = f2bf(b * c + a * sn);
    }
}

static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

static int launch_prologue(uint16_t *q, uint16_t *k, int ld, const float *wq, const float *wk,
                           const float *rope_cos, const float *rope_sin, int seq, int heads,
                           int head_dim, float eps, int split_half) {
    if (!require_device("head_norm_rope")) return IRIS_B200_ENODEV;
    if (seq <= 0 || heads <= 0) return IRIS_B200_OK;
    if (head_dim <= 0 || (head_dim & 1) || !q || !wq || !rope_cos || !rope_sin || (k && !wk)) {
        set_error(IRIS_B200_EINVAL, "head_norm_rope", "bad argument");
        return IRIS_B200_EINVAL;
    }
    bool fast = head_dim == 128 && ld % 8 == 0 && aligned16(q) && (!k || aligned16(k)) &&
                aligned16(rope_cos) && aligned16(rope_sin) && aligned16(wq) && (!k || aligned16(wk));
    if (fast) {
        long long units = (long long)seq * heads * (k ? 2 : 1);
        long long groups = (units + kUnroll - 1) / kUnroll;
        long long blocks = (groups * 16 + kThreads - 1) / kThreads;
        long long cap = (long long)g.sm_count * kBlocksPerSM;   /* one resident wave */
        if (blocks > cap) blocks = cap;
        if (split_half)
            k_head_norm_rope_128<true><<<(unsigned)blocks, kThreads, 0, g.stream>>>(
                q, k, ld, wq, wk, rope_cos, rope_sin, seq, heads, eps);
        else {
            long long segs = (long long)seq * (k ? 2 : 1);
            long long tb = (segs * 16 + kThreads - 1) / kThreads;
            if (tb > (long long)g.sm_count * kTokBlocksPerSM) tb = (long long)g.sm_count * kTokBlocksPerSM;
            k_head_norm_rope_128_tok<<<(unsigned)tb, kThreads, 0, g.stream>>>(
                q, k, ld, wq, wk, rope_cos, rope_sin, seq, heads, eps);
        }
        return after_launch("head_norm_rope") ? IRIS_B200_OK : IRIS_B200_ECUDA;
    }
    for (int pass = 0; pass < (k ? 2 : 1); pass++) {
        long long units = (long long)seq * heads;
        unsigned blocks = (unsigned)((units * 32 + 255) / 256);
        k_head_norm_rope_any<<<blocks, 256, 0, g.stream>>>(pass ? k : q, ld, pass ? wk : wq, rope_cos,
                                                           rope_sin, seq, heads, head_dim, eps, split_half);
        if (!after_launch("head_norm_rope")) return IRIS_B200_ECUDA;
    }
    return IRIS_B200_OK;
}

}  // namespace iris_b200

using namespace iris_b200;

extern "C" void iris_dev_head_norm_rope(uint16_t *x, int ld, const float *w,
                                        const float *rope_cos, const float *rope_sin,
                                        int seq, int heads, int head_dim, float eps,
                                        int split_half) {
    launch_prologue(x, NULL, ld, w, NULL, rope_cos, rope_sin, seq, heads, head_dim, eps, split_half);
}

extern "C" int iris_b200_qk_norm_rope(uint16_t *q, uint16_t *k, int ld,
                                      const float *wq, const float *wk,
                                      const float *rope_cos, const float *rope_sin,
                                      int seq, int heads, int head_dim, float eps, int split_half) {
    if (!k) {
        set_error(IRIS_B200_EINVAL, "qk_norm_rope", "k is NULL");
        return IRIS_B200_EINVAL;
    }
    return launch_prologue(q, k, ld, wq, wk, rope_cos, rope_sin, seq, heads, head_dim, eps, split_half);
}
