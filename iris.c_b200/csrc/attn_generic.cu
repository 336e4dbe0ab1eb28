/*
 * General attention kernel on CUDA cores: every argument combination of
 * iris_dev_attention (any head_dim up to 512, GQA, causal, key mask, any
 * alignment). It is the correctness path for the domains the tcgen05 kernel
 * does not take (the reference routes the same domains to cuBLAS + a softmax
 * kernel, iris_cuda.cu:897-936) and the on-device cross-check of that kernel.
 *
 * A block owns 8 consecutive queries of one head, one warp per query. Keys
 * are visited in tiles of 32 staged in shared memory; in a tile each lane
 * scores one key (full dot product against the query held in shared memory),
 * the warp does an online softmax over the 32 scores, then each lane
 * accumulates the output dims d = lane, lane + 32, ... Masked, causal-hidden
 * and out-of-range keys score -inf; a query with no valid key yields zeros
 * (iris_cuda.cu:811-812, :853).
 */
#include "common.cuh"

#include <math.h>

namespace iris_b200 {

static constexpr int kQPerBlock = 8;
static constexpr int kKeysPerTile = 32;
static constexpr int kMaxHeadDim = 512;

__global__ void __launch_bounds__(kQPerBlock * 32)
k_attention_generic(uint16_t *__restrict__ out, int ldo, const uint16_t *__restrict__ q,
                    const uint16_t *__restrict__ k, const uint16_t *__restrict__ v, int ldi,
                    int seq_q, int seq_k, int group, int head_dim, float scale_log2,
                    int causal, const int *__restrict__ key_mask) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kstride = head_dim + 2;                 /* odd word stride: no bank conflicts */
    uint16_t *ks = reinterpret_cast<uint16_t *>(smem_raw);
    uint16_t *vs = ks + kKeysPerTile * kstride;
    /* 32 (head_dim + 2) + 32 head_dim 16-bit elements precede it: a multiple of
     * four bytes for every head_dim, odd ones included. */
    float *qs = reinterpret_cast<float *>(vs + kKeysPerTile * head_dim);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, kvh = h / group;
    const int qi = blockIdx.x * kQPerBlock + warp;
    const bool qvalid = qi < seq_q;
    const int ndim = (head_dim + 31) / 32;            /* dims per lane, <= 16 */

    float *qrow = qs + warp * head_dim;
    for (int d = lane; d < head_dim; d += 32)
        qrow[d] = qvalid ? bf2f(q[(size_t)qi * ldi + (size_t)h * head_dim + d]) : 0.0f;

    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int t = 0; t < kMaxHeadDim / 32; t++) acc[t] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    /* Keys beyond the last query of the block are hidden from all its rows. */
    int kend = seq_k;
    if (causal) {
        int last = blockIdx.x * kQPerBlock + kQPerBlock;      /* exclusive */
        if (last < kend) kend = last;
    }
    const int limit = causal ? (qi + 1 < seq_k ? qi + 1 : seq_k) : seq_k;

    for (int k0 = 0; k0 < kend; k0 += kKeysPerTile) {
        __syncthreads();
        for (int i = threadIdx.x; i < kKeysPerTile * head_dim; i += blockDim.x) {
            int r = i / head_dim, d = i - r * head_dim;
            bool ok = k0 + r < seq_k;
            size_t off = (size_t)(k0 + r) * ldi + (size_t)kvh * head_dim + d;
            ks[r * kstride + d] = ok ? k[off] : (uint16_t)0;
            vs[r * head_dim + d] = ok ? v[off] : (uint16_t)0;
        }
        __syncthreads();

        int key = k0 + lane;
        bool valid = qvalid && key < limit && (!key_mask || key_mask[key] != 0);
        float dot = 0.0f;
        const uint16_t *kr = ks + lane * kstride;
        for (int d = 0; d < head_dim; d++) dot += qrow[d] * bf2f(kr[d]);
        float sc = valid ? dot * scale_log2 : -INFINITY;

        float mx = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float mnew = fmaxf(m, mx);
        float mref = mnew == -INFINITY ? 0.0f : mnew;          /* finite while nothing is valid */
        float alpha = exp2f(m - mref);
        float p = exp2f(sc - mref);
        float ps = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * alpha + ps;
        m = mnew;
        /* The tensor-core kernels round P to bf16 before P.V while the sum
         * keeps the unrounded value (iris_cuda.cu:819-831); same here. */
        float pb = bf2f(f2bf(p));
#pragma unroll
        for (int t = 0; t < kMaxHeadDim / 32; t++) acc[t] *= alpha;
        for (int j = 0; j < kKeysPerTile; j++) {
            float pj = __shfl_sync(0xffffffffu, pb, j);
            const uint16_t *vr = vs + j * head_dim;
#pragma unroll
            for (int t = 0; t < kMaxHeadDim / 32; t++) {
                int d = lane + 32 * t;
                if (t < ndim && d < head_dim) acc[t] += pj * bf2f(vr[d]);
            }
        }
    }
    if (!qvalid) return;
    float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int t = 0; t < kMaxHeadDim / 32; t++) {
        int d = lane + 32 * t;
        if (t < ndim && d < head_dim)
            out[(size_t)qi * ldo + (size_t)h * head_dim + d] = f2bf(acc[t] * inv);
    }
}

static size_t generic_smem(int head_dim) {
    return (size_t)kKeysPerTile * (head_dim + 2) * 2 + (size_t)kKeysPerTile * head_dim * 2 +
           (size_t)kQPerBlock * head_dim * 4;
}

int launch_attention_generic(uint16_t *out, int ldo, const uint16_t *q, const uint16_t *k,
                             const uint16_t *v, int ldi, int seq_q, int seq_k, int heads,
                             int kv_heads, int head_dim, float scale, int causal,
                             const int *key_mask) {
    if (head_dim > kMaxHeadDim) {
        set_error(IRIS_B200_EUNSUPPORTED, "attention", "head_dim above 512");
        return IRIS_B200_EUNSUPPORTED;
    }
    size_t smem = generic_smem(head_dim);
    if (smem > 48 * 1024) {
        if (!cuda_ok(cudaFuncSetAttribute(k_attention_generic, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)generic_smem(kMaxHeadDim)), "attention smem opt-in"))
            return IRIS_B200_ECUDA;
    }
    dim3 grid((seq_q + kQPerBlock - 1) / kQPerBlock, heads);
    k_attention_generic<<<grid, kQPerBlock * 32, smem, g.stream>>>(
        out, ldo, q, k, v, ldi, seq_q, seq_k, heads / kv_heads, head_dim,
        scale * 1.4426950408889634f, causal, key_mask);
    return after_launch("attention (generic)") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

}  // namespace iris_b200
