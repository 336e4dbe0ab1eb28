/* Shared state and helpers of the library's translation units. */
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "iris_b200.h"

namespace iris_b200 {

/* Global, single-device state (the reference keeps the same in file-scope
 * statics, iris_cuda.cu:74-92). */
struct State {
    int ready;
    int device;
    int owns_stream;
    cudaStream_t stream;
    cudaStream_t own_stream;
    char name[256];
    int sm_major, sm_minor, sm_count;
    int last_error;
    unsigned long long launches;
    cudaEvent_t t0, t1;
    /* pinned staging for uploads / downloads of pageable host memory */
    void *stage[2];
    cudaEvent_t stage_done[2];
    /* device status word written by kernels with bounded waits */
    unsigned int *dev_status;
    /* scratch for the host-pointer surface, grown on demand */
    void *scratch;
    size_t scratch_bytes;
};

extern State g;

void set_error(int code, const char *what, const char *detail);
/* Returns true when err is cudaSuccess; otherwise prints and records. */
bool cuda_ok(cudaError_t err, const char *what);
/* True when init has succeeded; otherwise records ENODEV and prints. */
bool require_device(const char *op);
/* Launch bookkeeping: counts the launch and records a launch failure. */
bool after_launch(const char *kernel);
/* Library scratch of at least `bytes` (NULL on failure). */
void *ensure_scratch(size_t bytes);

static constexpr size_t kStageBytes = (size_t)64 << 20;

/* bf16 <-> f32 with the reference's rounding: add 0x7FFF + lsb, truncate,
 * no NaN case (iris_cuda.cu:236-245). */
__device__ __forceinline__ float bf2f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) {
    uint32_t u = __float_as_uint(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16);
}
/* Hardware round-to-nearest-even pack; equal to pack_bf16x2 for every finite
 * input (lo in bits 0-15). */
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ float bf_lo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf_hi(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }

}  // namespace iris_b200
