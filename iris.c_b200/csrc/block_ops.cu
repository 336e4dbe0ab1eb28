/*
 * The row-wise operators either side of the attention path inside one
 * transformer block, and the FLUX.2 single-stream block assembled from them.
 *
 *   iris_dev_layer_norm_mod   LayerNorm without affine parameters, then
 *                             (1 + scale) and shift, fp32 in, bf16 out
 *                             (reference kernel: iris_cuda.cu:349-370)
 *   iris_dev_rms_norm(_mod)   RMSNorm with weight and optional (1 + scale),
 *                             fp32 in, bf16 out (iris_cuda.cu:372-386)
 *   iris_dev_rms_norm_residual  x += tanh(gate) * RMSNorm(a) * w in fp32
 *                             (iris_cuda.cu:388-400)
 *   iris_dev_swiglu           silu(gate) * up on bf16 column slices
 *                             (iris_cuda.cu:300-307)
 *   iris_dev_residual         x += gate * a in fp32 (iris_cuda.cu:309-314)
 *   iris_b200_double_block    the sequence the reference issues per double
 *                             block (iris_transformer_flux.c:3781-3823) in
 *                             seven launches instead of twenty-seven: every
 *                             launch covers the text and the image stream.
 *   iris_b200_zimage_block    the sequence of one Z-Image block
 *                             (iris_transformer_zimage.c:1940-1959) in nine
 *                             launches instead of twelve.
 *   iris_b200_single_block    the sequence the reference issues per single
 *                             block (iris_transformer_flux.c:3828-3845) in four
 *                             launches instead of eight: the projection
 *                             applies the Q/K prologue and SwiGLU in its
 *                             epilogue, and the output projection adds the
 *                             gated result to the hidden state in its epilogue.
 *
 * All three kernels are HBM-bound: every element is read once and written
 * once, 16 bytes per access.
 */
#include "common.cuh"

#include "iris_dev.h"
#include "kernels.h"

namespace iris_b200 {

namespace {

constexpr int kRowThreads = 256;
constexpr int kMaxSegments = 4;

/* Modulation by runs of rows: rows below end[i] (and not below end[i - 1])
 * take shift[i] / scale[i] (either may be NULL). */
struct RowMods {
    int n;
    int end[kMaxSegments];
    const float *shift[kMaxSegments];
    const float *scale[kMaxSegments];
};

__device__ __forceinline__ int segment_of(const RowMods &m, int row) {
    int i = 0;
    while (i + 1 < m.n && row >= m.end[i]) i++;
    return i;
}

__device__ __forceinline__ float block_sum(float v, float *sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                  /* sh may still be read from the previous reduction */
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; w++) t += sh[w];
    return t;
}

/* One block per row at a time, the row in registers (VPT float4 per thread,
 * so dims up to 1024 * VPT) between the three passes: mean, variance about
 * the mean (two-pass, as in the reference), output. Eight blocks per SM keep
 * enough loads in flight; one warp per row was measured slower (3.2 against
 * 4.8 TB/s at 4608 x 3072). */
template <int VPT>
__global__ void __launch_bounds__(kRowThreads, VPT <= 2 ? 8 : 6)
k_layer_norm_mod_rows(uint16_t *__restrict__ out, const float *__restrict__ x, const __grid_constant__ RowMods mods, int rows,
                      int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    const int nvec = dim >> 2;
    const float inv_dim = 1.0f / (float)dim;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * dim);
        uint2 *o = reinterpret_cast<uint2 *>(out + (size_t)row * dim);
        const int seg = segment_of(mods, row);
        const float *shift = mods.shift[seg], *scale = mods.scale[seg];
        float4 v[VPT];
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * kRowThreads;
            v[k] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
        const float mean = block_sum(s, sh) * inv_dim;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            if (threadIdx.x + k * kRowThreads < nvec) {
                const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
                q += (a * a + b * b) + (c * c + d * d);
            }
        }
        const float inv = rsqrtf(block_sum(q, sh) * inv_dim + eps);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * kRowThreads;
            if (i >= nvec) continue;
            float n[4] = {(v[k].x - mean) * inv, (v[k].y - mean) * inv, (v[k].z - mean) * inv, (v[k].w - mean) * inv};
            if (scale) {
                const float4 sc = reinterpret_cast<const float4 *>(scale)[i];
                n[0] *= 1.0f + sc.x; n[1] *= 1.0f + sc.y; n[2] *= 1.0f + sc.z; n[3] *= 1.0f + sc.w;
            }
            if (shift) {
                const float4 sf = reinterpret_cast<const float4 *>(shift)[i];
                n[0] += sf.x; n[1] += sf.y; n[2] += sf.z; n[3] += sf.w;
            }
            o[i] = make_uint2(cvt_bf16x2(n[0], n[1]), cvt_bf16x2(n[2], n[3]));
        }
    }
}

/* The same for the rows a rank owns of a hidden state that is sharded by rows
 * over several GPUs, with the all-gather in its stores: every output row goes
 * to the same row of every destination (this GPU's buffer and the peers',
 * plain 8-byte stores over NVLink), and the last block out advances this
 * rank's arrival word on every destination once all stores are visible at
 * system scope. The linear layer that follows on each GPU waits for those
 * words per row tile (gemm_sm100.cu: rows_arrived). */
template <int VPT>
__global__ void __launch_bounds__(kRowThreads, VPT <= 2 ? 8 : 6)
k_layer_norm_mod_gather(const __grid_constant__ GatherOut dst, const float *__restrict__ x, const float *__restrict__ shift,
                        const float *__restrict__ scale, int rows, int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    const int nvec = dim >> 2;
    const float inv_dim = 1.0f / (float)dim;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * dim);
        float4 v[VPT];
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * kRowThreads;
            v[k] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
        const float mean = block_sum(s, sh) * inv_dim;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            if (threadIdx.x + k * kRowThreads < nvec) {
                const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
                q += (a * a + b * b) + (c * c + d * d);
            }
        }
        const float inv = rsqrtf(block_sum(q, sh) * inv_dim + eps);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * kRowThreads;
            if (i >= nvec) continue;
            float n[4] = {(v[k].x - mean) * inv, (v[k].y - mean) * inv, (v[k].z - mean) * inv, (v[k].w - mean) * inv};
            if (scale) {
                const float4 sc = reinterpret_cast<const float4 *>(scale)[i];
                n[0] *= 1.0f + sc.x; n[1] *= 1.0f + sc.y; n[2] *= 1.0f + sc.z; n[3] *= 1.0f + sc.w;
            }
            if (shift) {
                const float4 sf = reinterpret_cast<const float4 *>(shift)[i];
                n[0] += sf.x; n[1] += sf.y; n[2] += sf.z; n[3] += sf.w;
            }
            const uint2 packed = make_uint2(cvt_bf16x2(n[0], n[1]), cvt_bf16x2(n[2], n[3]));
            for (int d = 0; d < dst.n; d++) reinterpret_cast<uint2 *>(dst.dst[d] + (size_t)row * dim)[i] = packed;
        }
    }
    /* this thread's rows are out before the block counts itself out */
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(dst.done, 1u);
        if (prev == gridDim.x - 1) {
            *dst.done = 0u;
            __threadfence_system();
            for (int d = 0; d < dst.n; d++)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst.word[d]), "r"(dst.seq) : "memory");
        }
    }
}

/* Any other row length: one block per row at a time, the row re-read from
 * L1 / L2 for each pass. */
__global__ void __launch_bounds__(kRowThreads)
k_layer_norm_mod_any(uint16_t *__restrict__ out, const float *__restrict__ x, const __grid_constant__ RowMods mods, int rows,
                     int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    const float inv_dim = 1.0f / (float)dim;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *xr = x + (size_t)row * dim;
        uint16_t *o = out + (size_t)row * dim;
        const int seg = segment_of(mods, row);
        const float *shift = mods.shift[seg], *scale = mods.scale[seg];
        float s = 0.0f;
        for (int i = threadIdx.x; i < dim; i += kRowThreads) s += xr[i];
        const float mean = block_sum(s, sh) * inv_dim;
        float q = 0.0f;
        for (int i = threadIdx.x; i < dim; i += kRowThreads) {
            const float d = xr[i] - mean;
            q += d * d;
        }
        const float inv = rsqrtf(block_sum(q, sh) * inv_dim + eps);
        for (int i = threadIdx.x; i < dim; i += kRowThreads) {
            float n = (xr[i] - mean) * inv;
            if (scale) n *= 1.0f + scale[i];
            if (shift) n += shift[i];
            o[i] = f2bf(n);
        }
    }
}

/* RMSNorm rows, one block per row at a time with the row in registers.
 * RESIDUAL false: out (bf16) = x * inv * w * (1 + scale); true: xres (fp32) +=
 * tanh(gate) * x * inv * w, where x is the projection result. scale / gate
 * may be NULL. */
template <int VPT, bool RESIDUAL>
__global__ void __launch_bounds__(kRowThreads, VPT <= 2 ? 8 : 6)
k_rms_norm_rows(uint16_t *__restrict__ out, float *__restrict__ xres, const float *__restrict__ x,
                const float *__restrict__ w, const float *__restrict__ mod, int rows, int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    const int nvec = dim >> 2;
    const float inv_dim = 1.0f / (float)dim;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * dim);
        float4 v[VPT];
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * kRowThreads;
            v[k] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
        }
        const float inv = rsqrtf(block_sum(s, sh) * inv_dim + eps);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int i = threadIdx.x + k * kRowThreads;
            if (i >= nvec) continue;
            const float4 w4 = reinterpret_cast<const float4 *>(w)[i];
            float n[4] = {v[k].x * inv * w4.x, v[k].y * inv * w4.y, v[k].z * inv * w4.z, v[k].w * inv * w4.w};
            if (RESIDUAL) {
                float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
                if (mod) {
                    const float4 m = reinterpret_cast<const float4 *>(mod)[i];
                    g = make_float4(tanhf(m.x), tanhf(m.y), tanhf(m.z), tanhf(m.w));
                }
                float4 *xo = reinterpret_cast<float4 *>(xres + (size_t)row * dim) + i;
                float4 xv = *xo;
                xv.x += g.x * n[0]; xv.y += g.y * n[1]; xv.z += g.z * n[2]; xv.w += g.w * n[3];
                *xo = xv;
            } else {
                if (mod) {
                    const float4 m = reinterpret_cast<const float4 *>(mod)[i];
                    n[0] *= 1.0f + m.x; n[1] *= 1.0f + m.y; n[2] *= 1.0f + m.z; n[3] *= 1.0f + m.w;
                }
                reinterpret_cast<uint2 *>(out + (size_t)row * dim)[i] = make_uint2(cvt_bf16x2(n[0], n[1]), cvt_bf16x2(n[2], n[3]));
            }
        }
    }
}

template <bool RESIDUAL>
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm_any(uint16_t *__restrict__ out, float *__restrict__ xres, const float *__restrict__ x, const float *__restrict__ w,
               const float *__restrict__ mod, int rows, int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *xr = x + (size_t)row * dim;
        float s = 0.0f;
        for (int i = threadIdx.x; i < dim; i += kRowThreads) s += xr[i] * xr[i];
        const float inv = rsqrtf(block_sum(s, sh) / (float)dim + eps);
        for (int i = threadIdx.x; i < dim; i += kRowThreads) {
            const float n = xr[i] * inv * w[i];
            if (RESIDUAL) xres[(size_t)row * dim + i] += (mod ? tanhf(mod[i]) : 1.0f) * n;
            else out[(size_t)row * dim + i] = f2bf(mod ? n * (1.0f + mod[i]) : n);
        }
    }
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

/* Eight columns per thread when the slices allow 16-byte accesses. */
__global__ void __launch_bounds__(256)
k_swiglu8(uint16_t *__restrict__ out, int ldo, const uint16_t *__restrict__ gate, const uint16_t *__restrict__ up, int ldi,
          int cols8, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols8, c = (i - r * cols8) * 8;
        const uint4 gv = *reinterpret_cast<const uint4 *>(gate + r * ldi + c);
        const uint4 uv = *reinterpret_cast<const uint4 *>(up + r * ldi + c);
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            ow[k] = cvt_bf16x2(silu_mul(bf_lo(gw[k]), bf_lo(uw[k])), silu_mul(bf_hi(gw[k]), bf_hi(uw[k])));
        *reinterpret_cast<uint4 *>(out + r * ldo + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

__global__ void __launch_bounds__(256)
k_swiglu1(uint16_t *out, int ldo, const uint16_t *gate, const uint16_t *up, int ldi, int cols, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols, c = i - r * cols;
        out[r * ldo + c] = f2bf(silu_mul(bf2f(gate[r * ldi + c]), bf2f(up[r * ldi + c])));
    }
}

__global__ void __launch_bounds__(256)
k_residual4(float *__restrict__ x, const float *__restrict__ a, const float *__restrict__ gate, int dim4, size_t n4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 xv = reinterpret_cast<float4 *>(x)[i];
        const float4 av = reinterpret_cast<const float4 *>(a)[i];
        float4 g4 = make_float4(1.f, 1.f, 1.f, 1.f);
        if (gate) g4 = reinterpret_cast<const float4 *>(gate)[i % dim4];
        xv.x += g4.x * av.x; xv.y += g4.y * av.y; xv.z += g4.z * av.z; xv.w += g4.w * av.w;
        reinterpret_cast<float4 *>(x)[i] = xv;
    }
}

__global__ void __launch_bounds__(256)
k_residual1(float *x, const float *a, const float *gate, int dim, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] += (gate ? gate[i % dim] : 1.0f) * a[i];
}

unsigned blocks_for(size_t items, int per_block, int per_sm) {
    size_t b = (items + per_block - 1) / per_block;
    const size_t cap = (size_t)g.sm_count * per_sm;
    if (b > cap) b = cap;
    return (unsigned)(b ? b : 1);
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

int layer_norm_mods(uint16_t *out, const float *x, const RowMods &mods, int rows, int dim, float eps) {
    if (!require_device("layer_norm_mod")) return IRIS_B200_ENODEV;
    if (!out || !x || rows < 0 || dim <= 0 || mods.n < 1 || mods.n > kMaxSegments) {
        set_error(IRIS_B200_EINVAL, "layer_norm_mod", "bad argument");
        return IRIS_B200_EINVAL;
    }
    if (rows == 0) return IRIS_B200_OK;
    const int nvec = dim / 4;
    bool vec = dim % 4 == 0 && nvec <= 4 * kRowThreads && aligned16(x) && ((uintptr_t)out & 7) == 0;
    for (int i = 0; i < mods.n; i++) vec = vec && aligned16(mods.shift[i]) && aligned16(mods.scale[i]);
    if (vec) {
        const unsigned grid = blocks_for((size_t)rows, 1, 8);
#define IRIS_LN_LAUNCH(VPT) k_layer_norm_mod_rows<VPT><<<grid, kRowThreads, 0, g.stream>>>(out, x, mods, rows, dim, eps)
        if (nvec <= kRowThreads) IRIS_LN_LAUNCH(1);
        else if (nvec <= 2 * kRowThreads) IRIS_LN_LAUNCH(2);
        else if (nvec <= 3 * kRowThreads) IRIS_LN_LAUNCH(3);
        else IRIS_LN_LAUNCH(4);
#undef IRIS_LN_LAUNCH
    } else {
        k_layer_norm_mod_any<<<blocks_for((size_t)rows, 1, 8), kRowThreads, 0, g.stream>>>(out, x, mods, rows, dim, eps);
    }
    return after_launch("k_layer_norm_mod") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

int layer_norm_mod(uint16_t *out, const float *x, const float *shift, const float *scale, int rows, int dim, float eps) {
    RowMods m = {};
    m.n = 1;
    m.end[0] = rows;
    m.shift[0] = shift;
    m.scale[0] = scale;
    return layer_norm_mods(out, x, m, rows, dim, eps);
}

template <bool RESIDUAL>
int rms_norm_rows(uint16_t *out, float *xres, const float *x, const float *w, const float *mod, int rows, int dim, float eps,
                  const char *op) {
    if (!require_device(op)) return IRIS_B200_ENODEV;
    if ((RESIDUAL ? !xres : !out) || !x || !w || rows < 0 || dim <= 0) {
        set_error(IRIS_B200_EINVAL, op, "bad argument");
        return IRIS_B200_EINVAL;
    }
    if (rows == 0) return IRIS_B200_OK;
    const int nvec = dim / 4;
    const bool vec = dim % 4 == 0 && nvec <= 4 * kRowThreads && aligned16(x) && aligned16(w) && aligned16(mod) &&
                     aligned16(xres) && ((uintptr_t)out & 7) == 0;
    if (vec) {
        const unsigned grid = blocks_for((size_t)rows, 1, 8);
#define IRIS_RMS_LAUNCH(VPT) \
    k_rms_norm_rows<VPT, RESIDUAL><<<grid, kRowThreads, 0, g.stream>>>(out, xres, x, w, mod, rows, dim, eps)
        if (nvec <= kRowThreads) IRIS_RMS_LAUNCH(1);
        else if (nvec <= 2 * kRowThreads) IRIS_RMS_LAUNCH(2);
        else if (nvec <= 3 * kRowThreads) IRIS_RMS_LAUNCH(3);
        else IRIS_RMS_LAUNCH(4);
#undef IRIS_RMS_LAUNCH
    } else {
        k_rms_norm_any<RESIDUAL><<<blocks_for((size_t)rows, 1, 8), kRowThreads, 0, g.stream>>>(out, xres, x, w, mod, rows, dim, eps);
    }
    return after_launch("k_rms_norm") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

}  // namespace

int launch_layer_norm_mod_gather(const GatherOut &out, const float *x, const float *shift, const float *scale, int rows,
                                 int dim, float eps) {
    if (!require_device("layer_norm_mod (gather)")) return IRIS_B200_ENODEV;
    const int nvec = dim / 4;
    bool ok = x && rows >= 0 && dim > 0 && out.n >= 1 && out.n <= 16 && out.done && dim % 4 == 0 && nvec <= 4 * kRowThreads &&
              aligned16(x) && aligned16(shift) && aligned16(scale);
    for (int d = 0; ok && d < out.n; d++) ok = out.dst[d] && out.word[d] && ((uintptr_t)out.dst[d] & 7) == 0;
    if (!ok) {
        set_error(IRIS_B200_EINVAL, "layer_norm_mod (gather)", "bad argument (dim a multiple of 4 up to 4096, aligned operands)");
        return IRIS_B200_EINVAL;
    }
    /* rows == 0 still has to announce itself: one block, no rows */
    const unsigned grid = blocks_for((size_t)(rows > 0 ? rows : 1), 1, 8);
    if (nvec <= kRowThreads) k_layer_norm_mod_gather<1><<<grid, kRowThreads, 0, g.stream>>>(out, x, shift, scale, rows, dim, eps);
    else if (nvec <= 2 * kRowThreads) k_layer_norm_mod_gather<2><<<grid, kRowThreads, 0, g.stream>>>(out, x, shift, scale, rows, dim, eps);
    else if (nvec <= 3 * kRowThreads) k_layer_norm_mod_gather<3><<<grid, kRowThreads, 0, g.stream>>>(out, x, shift, scale, rows, dim, eps);
    else k_layer_norm_mod_gather<4><<<grid, kRowThreads, 0, g.stream>>>(out, x, shift, scale, rows, dim, eps);
    return after_launch("k_layer_norm_mod_gather") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

namespace {

int swiglu(uint16_t *out, int ldo, const uint16_t *gate, const uint16_t *up, int ldi, int rows, int cols) {
    if (!require_device("swiglu")) return IRIS_B200_ENODEV;
    if (!out || !gate || !up || rows < 0 || cols < 0 || ldo < cols || ldi < cols) {
        set_error(IRIS_B200_EINVAL, "swiglu", "bad argument");
        return IRIS_B200_EINVAL;
    }
    const size_t n = (size_t)rows * cols;
    if (n == 0) return IRIS_B200_OK;
    if (cols % 8 == 0 && ldo % 8 == 0 && ldi % 8 == 0 && aligned16(out) && aligned16(gate) && aligned16(up))
        k_swiglu8<<<blocks_for(n / 8, 256, 8), 256, 0, g.stream>>>(out, ldo, gate, up, ldi, cols / 8, n / 8);
    else
        k_swiglu1<<<blocks_for(n, 256, 8), 256, 0, g.stream>>>(out, ldo, gate, up, ldi, cols, n);
    return after_launch("k_swiglu") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

int residual(float *x, const float *a, const float *gate, int rows, int dim) {
    if (!require_device("residual")) return IRIS_B200_ENODEV;
    if (!x || !a || rows < 0 || dim <= 0) {
        set_error(IRIS_B200_EINVAL, "residual", "bad argument");
        return IRIS_B200_EINVAL;
    }
    const size_t n = (size_t)rows * dim;
    if (n == 0) return IRIS_B200_OK;
    if (dim % 4 == 0 && aligned16(x) && aligned16(a) && aligned16(gate))
        k_residual4<<<blocks_for(n / 4, 256, 8), 256, 0, g.stream>>>(x, a, gate, dim / 4, n / 4);
    else
        k_residual1<<<blocks_for(n, 256, 8), 256, 0, g.stream>>>(x, a, gate, dim, n);
    return after_launch("k_residual") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

}  // namespace

}  // namespace iris_b200

using namespace iris_b200;

extern "C" void iris_dev_layer_norm_mod(uint16_t *out, const float *x, const float *shift, const float *scale, int rows,
                                        int dim, float eps) {
    layer_norm_mod(out, x, shift, scale, rows, dim, eps);
}

extern "C" void iris_dev_rms_norm(uint16_t *out, const float *x, const float *w, int rows, int dim, float eps) {
    rms_norm_rows<false>(out, NULL, x, w, NULL, rows, dim, eps, "rms_norm");
}

extern "C" void iris_dev_rms_norm_mod(uint16_t *out, const float *x, const float *w, const float *scale, int rows, int dim,
                                      float eps) {
    rms_norm_rows<false>(out, NULL, x, w, scale, rows, dim, eps, "rms_norm_mod");
}

extern "C" void iris_dev_rms_norm_residual(float *x, const float *a, const float *w, const float *gate, int rows, int dim,
                                           float eps) {
    rms_norm_rows<true>(NULL, x, a, w, gate, rows, dim, eps, "rms_norm_residual");
}

extern "C" void iris_dev_swiglu(uint16_t *out, int ldo, const uint16_t *gate, const uint16_t *up, int ldi, int rows,
                                int cols) {
    swiglu(out, ldo, gate, up, ldi, rows, cols);
}

extern "C" void iris_dev_residual(float *x, const float *a, const float *gate, int rows, int dim) {
    residual(x, a, gate, rows, dim);
}

extern "C" size_t iris_b200_single_block_scratch_bytes(int seq, int dim, int mlp) {
    if (seq < 0 || dim <= 0 || mlp <= 0) return 0;
    /* norm [seq, dim] | qkv [seq, 3 dim] | cat [seq, dim + mlp], bf16, each 256-byte aligned */
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    return up256((size_t)seq * dim * 2) + up256((size_t)seq * 3 * dim * 2) + up256((size_t)seq * ((size_t)dim + mlp) * 2);
}

extern "C" int iris_b200_single_block_segments(float *x, void *scratch, const uint16_t *w_in, const uint16_t *w_out,
                                               const float *norm_q, const float *norm_k, const iris_b200_segment *segs,
                                               int nsegs, const float *rope_cos, const float *rope_sin, int seq, int dim,
                                               int heads, int mlp, float eps, const int *key_mask) {
    if (!require_device("single_block")) return IRIS_B200_ENODEV;
    bool ok = x && scratch && w_in && w_out && norm_q && norm_k && segs && nsegs >= 1 && nsegs <= kMaxSegments && rope_cos &&
              rope_sin && seq >= 0 && dim > 0 && heads > 0 && mlp > 0 && dim == heads * 128 && ((uintptr_t)scratch & 255) == 0;
    /* the segments follow one another and cover the rows */
    int next = 0;
    for (int i = 0; ok && i < nsegs; i++) {
        ok = segs[i].start == next && segs[i].len >= 0 && segs[i].mod;
        next += segs[i].len;
    }
    if (!ok || next != seq) {
        set_error(IRIS_B200_EINVAL, "single_block",
                  dim > 0 && dim != heads * 128 ? "head_dim must be 128" : "bad argument, or segments that do not tile the rows");
        return IRIS_B200_EINVAL;
    }
    if (seq == 0) return IRIS_B200_OK;
    const int ldc = dim + mlp;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    unsigned char *base = static_cast<unsigned char *>(scratch);
    uint16_t *norm = reinterpret_cast<uint16_t *>(base);
    uint16_t *qkv = reinterpret_cast<uint16_t *>(base + up256((size_t)seq * dim * 2));
    uint16_t *cat = reinterpret_cast<uint16_t *>(base + up256((size_t)seq * dim * 2) + up256((size_t)seq * 3 * dim * 2));
    RowMods mods = {};
    int seg_end[kMaxSegments];
    const float *seg_gate[kMaxSegments];
    mods.n = nsegs;
    for (int i = 0; i < nsegs; i++) {
        mods.end[i] = seg_end[i] = segs[i].start + segs[i].len;
        mods.shift[i] = segs[i].mod;
        mods.scale[i] = segs[i].mod + dim;
        seg_gate[i] = segs[i].mod + 2 * dim;
    }
    int rc = layer_norm_mods(norm, x, mods, seq, dim, eps);
    if (rc != IRIS_B200_OK) return rc;
    /* Q, K (normalised, rotated) and V to qkv; silu(gate) * up straight into the MLP half of cat */
    rc = iris_b200_linear_glu(qkv, 3 * dim, cat + dim, ldc, norm, w_in, seq, dim, heads, mlp, norm_q, norm_k, rope_cos,
                              rope_sin, eps);
    if (rc != IRIS_B200_OK) return rc;
    iris_b200_clear_error();
    iris_dev_attention(cat, ldc, qkv, qkv + dim, qkv + 2 * dim, 3 * dim, seq, seq, heads, heads, 128, 0.08838834764831845f, 0,
                       key_mask);
    rc = iris_b200_last_error();
    if (rc != IRIS_B200_OK) return rc;
    return launch_linear_residual_segments(x, dim, cat, ldc, w_out, ldc, seg_end, seg_gate, nsegs, seq, ldc, dim);
}

extern "C" int iris_b200_single_block(float *x, void *scratch, const uint16_t *w_in, const uint16_t *w_out,
                                      const float *norm_q, const float *norm_k, const float *mod,
                                      const float *rope_cos, const float *rope_sin, int seq, int dim, int heads,
                                      int mlp, const int *key_mask) {
    const iris_b200_segment all = {0, seq, mod};
    return iris_b200_single_block_segments(x, scratch, w_in, w_out, norm_q, norm_k, mod ? &all : NULL, 1, rope_cos, rope_sin,
                                           seq, dim, heads, mlp, 1e-6f, key_mask);
}

/* norm [seq, dim] | qkv [seq, 3 dim] | cat [seq, max(dim, mlp)], bf16 */
extern "C" size_t iris_b200_double_block_scratch_bytes(int seq, int dim, int mlp) {
    if (seq < 0 || dim <= 0 || mlp <= 0) return 0;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t ldc = dim > mlp ? dim : mlp;
    return up256((size_t)seq * dim * 2) + up256((size_t)seq * 3 * dim * 2) + up256((size_t)seq * ldc * 2);
}

extern "C" int iris_b200_double_block(float *x, void *scratch, const iris_b200_stream_weights *txt,
                                      const iris_b200_stream_weights *img, const float *rope_cos,
                                      const float *rope_sin, int seq, int txt_seq, int dim, int heads, int mlp,
                                      const int *key_mask) {
    if (!require_device("double_block")) return IRIS_B200_ENODEV;
    bool ok = x && scratch && txt && img && rope_cos && rope_sin && seq >= 0 && txt_seq >= 0 && txt_seq <= seq && dim > 0 &&
              heads > 0 && mlp > 0 && dim == heads * 128 && ((uintptr_t)scratch & 255) == 0;
    const iris_b200_stream_weights *sw[2] = {txt, img};
    for (int m = 0; m < 2 && ok; m++)
        ok = sw[m]->qkv && sw[m]->proj && sw[m]->ff_in && sw[m]->ff_out && sw[m]->norm_q && sw[m]->norm_k && sw[m]->mod;
    if (!ok) {
        set_error(IRIS_B200_EINVAL, "double_block", dim > 0 && dim != heads * 128 ? "head_dim must be 128" : "bad argument");
        return IRIS_B200_EINVAL;
    }
    if (seq == 0) return IRIS_B200_OK;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    unsigned char *base = static_cast<unsigned char *>(scratch);
    uint16_t *norm = reinterpret_cast<uint16_t *>(base);
    uint16_t *h = reinterpret_cast<uint16_t *>(base + up256((size_t)seq * dim * 2));
    uint16_t *cat = reinterpret_cast<uint16_t *>(base + up256((size_t)seq * dim * 2) + up256((size_t)seq * 3 * dim * 2));
    const float eps = 1e-6f;
    const float *tm = txt->mod, *im = img->mod;
    int rc;
    /* attention half: both streams in every launch, text rows first */
    RowMods m1 = {};
    m1.n = 2;
    m1.end[0] = txt_seq;
    m1.end[1] = seq;
    m1.shift[0] = tm;
    m1.scale[0] = tm + dim;
    m1.shift[1] = im;
    m1.scale[1] = im + dim;
    if ((rc = layer_norm_mods(norm, x, m1, seq, dim, eps))) return rc;
    TwoStreamLinear l = {};
    l.x = norm;
    l.ldx = l.ldw = l.in = dim;
    l.W[0] = txt->qkv;
    l.W[1] = img->qkv;
    l.rows = seq;
    l.split = txt_seq;
    l.qkv = h;
    l.ldy = 3 * dim;
    l.heads = heads;
    l.wq[0] = txt->norm_q;
    l.wq[1] = img->norm_q;
    l.wk[0] = txt->norm_k;
    l.wk[1] = img->norm_k;
    l.rope_cos = rope_cos;
    l.rope_sin = rope_sin;
    l.eps = eps;
    if ((rc = launch_linear_two(l))) return rc;
    iris_b200_clear_error();
    iris_dev_attention(cat, dim, h, h + dim, h + 2 * dim, 3 * dim, seq, seq, heads, heads, 128, 0.08838834764831845f, 0,
                       key_mask);
    if ((rc = iris_b200_last_error()) != IRIS_B200_OK) return rc;
    TwoStreamLinear o = {};
    o.x = cat;
    o.ldx = o.ldw = o.in = dim;
    o.W[0] = txt->proj;
    o.W[1] = img->proj;
    o.rows = seq;
    o.split = txt_seq;
    o.out = dim;
    o.y32 = x;
    o.ldy = dim;
    o.gate[0] = tm + 2 * dim;
    o.gate[1] = im + 2 * dim;
    if ((rc = launch_linear_two(o))) return rc;
    /* feed-forward half: the gate | up projection stores silu(gate) * up */
    RowMods m2 = m1;
    m2.shift[0] = tm + 3 * dim;
    m2.scale[0] = tm + 4 * dim;
    m2.shift[1] = im + 3 * dim;
    m2.scale[1] = im + 4 * dim;
    if ((rc = layer_norm_mods(norm, x, m2, seq, dim, eps))) return rc;
    TwoStreamLinear f = {};
    f.x = norm;
    f.ldx = f.ldw = f.in = dim;
    f.W[0] = txt->ff_in;
    f.W[1] = img->ff_in;
    f.rows = seq;
    f.split = txt_seq;
    f.act = cat;
    f.lda = f.mlp = mlp;
    if ((rc = launch_linear_two(f))) return rc;
    TwoStreamLinear d = {};
    d.x = cat;
    d.ldx = d.ldw = d.in = mlp;
    d.W[0] = txt->ff_out;
    d.W[1] = img->ff_out;
    d.rows = seq;
    d.split = txt_seq;
    d.out = dim;
    d.y32 = x;
    d.ldy = dim;
    d.gate[0] = tm + 5 * dim;
    d.gate[1] = im + 5 * dim;
    return launch_linear_two(d);
}

/* norm [seq, dim] | qkv [seq, 3 dim] | act [seq, max(dim, ff)] bf16, then the projection result [seq, dim] fp32 */
extern "C" size_t iris_b200_zimage_block_scratch_bytes(int seq, int dim, int ff) {
    if (seq < 0 || dim <= 0 || ff <= 0) return 0;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t lda = dim > ff ? dim : ff;
    return up256((size_t)seq * dim * 2) + up256((size_t)seq * 3 * dim * 2) + up256((size_t)seq * lda * 2) +
           up256((size_t)seq * dim * 4);
}

extern "C" int iris_b200_zimage_block(float *x, void *scratch, const iris_b200_zimage_weights *w, const float *mod,
                                      const float *rope_cos, const float *rope_sin, int seq, int dim, int heads, int ff,
                                      const int *key_mask) {
    if (!require_device("zimage_block")) return IRIS_B200_ENODEV;
    const bool ok = x && scratch && w && w->qkv && w->proj && w->ff_in && w->ff_out && w->norm_q && w->norm_k && w->attn_norm1 &&
                    w->attn_norm2 && w->ffn_norm1 && w->ffn_norm2 && rope_cos && rope_sin && seq >= 0 && dim > 0 && heads > 0 &&
                    ff > 0 && dim == heads * 128 && ((uintptr_t)scratch & 255) == 0;
    if (!ok) {
        set_error(IRIS_B200_EINVAL, "zimage_block", dim > 0 && dim != heads * 128 ? "head_dim must be 128" : "bad argument");
        return IRIS_B200_EINVAL;
    }
    if (seq == 0) return IRIS_B200_OK;
    auto up256 = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t lda = dim > ff ? dim : ff;
    unsigned char *base = static_cast<unsigned char *>(scratch);
    uint16_t *norm = reinterpret_cast<uint16_t *>(base);
    base += up256((size_t)seq * dim * 2);
    uint16_t *qkv = reinterpret_cast<uint16_t *>(base);
    base += up256((size_t)seq * 3 * dim * 2);
    uint16_t *act = reinterpret_cast<uint16_t *>(base);
    base += up256((size_t)seq * lda * 2);
    float *out = reinterpret_cast<float *>(base);
    const float eps = 1e-5f;                    /* ZI_NORM_EPS, iris_transformer_zimage.c:47 */
    int rc;
    if ((rc = rms_norm_rows<false>(norm, NULL, x, w->attn_norm1, mod, seq, dim, eps, "rms_norm_mod"))) return rc;
    rc = iris_b200_linear_qk_norm_rope(qkv, 3 * dim, norm, w->qkv, seq, dim, 3 * dim, heads, w->norm_q, w->norm_k, rope_cos,
                                       rope_sin, eps);
    if (rc != IRIS_B200_OK) return rc;
    iris_b200_clear_error();
    iris_dev_attention(act, dim, qkv, qkv + dim, qkv + 2 * dim, 3 * dim, seq, seq, heads, heads, 128, 0.08838834764831845f, 0,
                       key_mask);
    if ((rc = iris_b200_last_error()) != IRIS_B200_OK) return rc;
    iris_dev_linear_f32(out, act, w->proj, seq, dim, dim);
    if ((rc = iris_b200_last_error()) != IRIS_B200_OK) return rc;
    if ((rc = rms_norm_rows<true>(NULL, x, out, w->attn_norm2, mod ? mod + dim : NULL, seq, dim, eps, "rms_norm_residual")))
        return rc;
    if ((rc = rms_norm_rows<false>(norm, NULL, x, w->ffn_norm1, mod ? mod + 2 * dim : NULL, seq, dim, eps, "rms_norm_mod")))
        return rc;
    rc = iris_b200_linear_glu(NULL, 0, act, ff, norm, w->ff_in, seq, dim, 0, ff, NULL, NULL, NULL, NULL, eps);
    if (rc != IRIS_B200_OK) return rc;
    iris_dev_linear_f32(out, act, w->ff_out, seq, ff, dim);
    if ((rc = iris_b200_last_error()) != IRIS_B200_OK) return rc;
    return rms_norm_rows<true>(NULL, x, out, w->ffn_norm2, mod ? mod + 3 * dim : NULL, seq, dim, eps, "rms_norm_residual");
}
