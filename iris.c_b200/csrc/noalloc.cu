/*
 * Split-K attention for callers that must not allocate device memory.
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they
 * run attention: a real-time render or audio thread that may not block on the
 * driver's allocator lock, a process whose memory budget was handed out in
 * full at start-up (a fixed arena owned by another runtime), or code running
 * between graph launches that has promised not to touch the allocator. The
 * ordinary chunked attention needs a carried state in global memory
 * (normalised fp32 output + log2-sum-exp per row) that somebody has to
 * allocate; here that state lives in a fixed array that is part of the
 * library image, so the call allocates nothing.
 *
 * Cost and limits: the array occupies kStateFloats * 4 bytes (16.1 MiB) on
 * every GPU that loads the library, until the process exits. Problems whose
 * state does not fit are rejected. All calls share the one array: two calls
 * whose kernels overlap on the GPU (different streams, different host
 * threads) race on it; calls on the library's single stream are ordered and
 * safe. Nothing in the array has to start at zero: the first chunk of every
 * call overwrites the state of every row it later reads.
 */
#include "common.cuh"

#include "kernels.h"

using namespace iris_b200;

namespace {

constexpr size_t kMaxOutFloats = (size_t)4 << 20;            /* seq_q * heads * 128 <= 4 Mi */
constexpr size_t kMaxLseFloats = kMaxOutFloats / 128;        /* seq_q * heads */
constexpr size_t kStateFloats = kMaxOutFloats + kMaxLseFloats;

/* The scratch itself. In host code this name is only a handle for the
 * runtime, not a device address. */
static __device__ __align__(256) float g_state[kStateFloats];

constexpr int kMaxDevices = 64;
float *g_state_ptr[kMaxDevices];

/* Device address of g_state on the current device, looked up once per device. */
float *state_address(void) {
    int dev = -1;
    if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice") || dev < 0 || dev >= kMaxDevices) return NULL;
    if (!g_state_ptr[dev]) {
        void *ptr = NULL;
        if (!cuda_ok(cudaGetSymbolAddress(&ptr, g_state), "cudaGetSymbolAddress")) return NULL;
        g_state_ptr[dev] = static_cast<float *>(ptr);
    }
    return g_state_ptr[dev];
}

}  // namespace

extern "C" size_t iris_b200_attention_noalloc_max_elems(void) { return kMaxOutFloats; }

extern "C" int iris_b200_attention_noalloc(uint16_t *out, int ldo,
                                           const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                           int ldi, int seq_q, int seq_k, int heads, float scale,
                                           int nsplit) {
    if (!require_device("attention_noalloc")) return IRIS_B200_ENODEV;
    if (!out || seq_k <= 0 || nsplit < 1) {
        set_error(IRIS_B200_EINVAL, "attention_noalloc", "bad argument");
        return IRIS_B200_EINVAL;
    }
    int rc = check_attention_args("attention_noalloc", out, q, k, v, ldo, ldi, ldi, seq_q, seq_k, heads, heads, 128);
    if (rc != IRIS_B200_OK) return rc;
    if ((size_t)seq_q * heads * 128 > kMaxOutFloats) {
        char msg[160];
        snprintf(msg, sizeof(msg), "seq_q * heads * 128 = %zu exceeds the built-in scratch of %zu elements",
                 (size_t)seq_q * heads * 128, kMaxOutFloats);
        set_error(IRIS_B200_EINVAL, "attention_noalloc", msg);
        return IRIS_B200_EINVAL;
    }
    if (!sm100_supported(out, ldo, q, k, v, ldi, heads, heads, 128, 0, scale)) {
        set_error(IRIS_B200_EUNSUPPORTED, "attention_noalloc", "arguments outside the tcgen05 kernel's domain");
        return IRIS_B200_EUNSUPPORTED;
    }
    if (seq_q == 0) return IRIS_B200_OK;
    float *state = state_address();
    if (!state) return IRIS_B200_ECUDA;
    float *o_state = state, *lse_state = state + kMaxOutFloats;
    /* Key chunks of whole 128-key tiles, as even as they come. */
    int tiles = (seq_k + 127) / 128;
    if (nsplit > tiles) nsplit = tiles;
    int done = 0;
    for (int i = 0; i < nsplit; i++) {
        int t1 = (int)((long long)tiles * (i + 1) / nsplit);
        int k0 = done * 128, k1 = t1 * 128 < seq_k ? t1 * 128 : seq_k;
        done = t1;
        int mode = nsplit == 1 ? 0 : (i == 0 ? 1 : (i == nsplit - 1 ? 3 : 2));
        AttnArgs a = attn_args(out, ldo, q, ldi, k + (size_t)k0 * ldi, v + (size_t)k0 * ldi, ldi, seq_q, k1 - k0,
                               heads, scale, NULL);
        a.acc_mode = mode;
        a.o_acc = o_state;
        a.lse_acc = lse_state;
        a.max_parts = 1;
        a.no_scratch = true;        /* the library's own scratch would have to be allocated */
        rc = launch_attention_sm100(a);
        if (rc != IRIS_B200_OK) return rc;
    }
    return IRIS_B200_OK;
}
