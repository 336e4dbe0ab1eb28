/*
 * Runtime of the device surface: init / cleanup, memory, copies, status,
 * stream sharing and the event stopwatch.
 *
 * Behaviour follows the reference runtime (iris_cuda.cu:117-230): one
 * stream, blocking uploads through two pinned staging buffers, blocking
 * download, free() that first waits for the stream, errors printed as
 * "iris_dev: <what> failed: <why>".
 */
#include "common.cuh"

#include <string.h>

#include "iris_dev.h"
#include "kernels.h"

namespace iris_b200 {

State g = {};

void set_error(int code, const char *what, const char *detail) {
    fprintf(stderr, "iris_dev: %s failed: %s\n", what, detail ? detail : iris_b200_strerror(code));
    if (g.last_error == IRIS_B200_OK) g.last_error = code;
}

bool cuda_ok(cudaError_t err, const char *what) {
    if (err == cudaSuccess) return true;
    set_error(IRIS_B200_ECUDA, what, cudaGetErrorString(err));
    return false;
}

bool require_device(const char *op) {
    if (g.ready) return true;
    set_error(IRIS_B200_ENODEV, op, "device not initialised (iris_dev_init)");
    return false;
}

bool after_launch(const char *kernel) {
    g.launches++;
    return cuda_ok(cudaGetLastError(), kernel);
}

void *ensure_scratch(size_t bytes) {
    if (bytes <= g.scratch_bytes) return g.scratch;
    if (g.scratch) {
        cuda_ok(cudaStreamSynchronize(g.stream), "sync");
        cuda_ok(cudaFree(g.scratch), "free");
    }
    g.scratch = NULL;
    g.scratch_bytes = 0;
    if (cudaMalloc(&g.scratch, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error(IRIS_B200_ENOMEM, "scratch allocation", NULL);
        g.scratch = NULL;
        return NULL;
    }
    g.scratch_bytes = bytes;
    return g.scratch;
}

__global__ void k_f32_to_bf16(uint16_t *dst, const float *src, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = f2bf(src[i]);
}

}  // namespace iris_b200

using namespace iris_b200;

extern "C" {

int iris_b200_last_error(void) { return g.last_error; }
void iris_b200_clear_error(void) { g.last_error = IRIS_B200_OK; }

const char *iris_b200_strerror(int code) {
    switch (code) {
    case IRIS_B200_OK: return "ok";
    case IRIS_B200_EINVAL: return "invalid argument";
    case IRIS_B200_ECUDA: return "CUDA call failed";
    case IRIS_B200_ETIMEOUT: return "bounded wait inside a kernel ran out";
    case IRIS_B200_ENODEV: return "device not initialised";
    case IRIS_B200_ENOMEM: return "device allocation failed";
    case IRIS_B200_EUNSUPPORTED: return "no kernel for this argument combination";
    case IRIS_B200_ECOMM: return "collective transport failed";
    }
    return "unknown error";
}

int iris_b200_set_device(int ordinal) {
    if (g.ready || ordinal < 0) return IRIS_B200_EINVAL;
    g.device = ordinal;
    return IRIS_B200_OK;
}

int iris_dev_init(void) {
    if (g.ready) return 1;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= g.device) {
        (void)cudaGetLastError();
        return 0;
    }
    if (cudaSetDevice(g.device) != cudaSuccess) return 0;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, g.device) != cudaSuccess) return 0;
    snprintf(g.name, sizeof(g.name), "%s", prop.name);
    g.sm_major = prop.major;
    g.sm_minor = prop.minor;
    g.sm_count = prop.multiProcessorCount;
    /* The kernels are built for sm_100a only: there is no other code path. */
    if (prop.major != 10) {
        fprintf(stderr, "iris_dev: %s is sm_%d%d, this library needs sm_100\n", prop.name,
                prop.major, prop.minor);
        return 0;
    }
    if (cudaStreamCreateWithFlags(&g.own_stream, cudaStreamNonBlocking) != cudaSuccess) return 0;
    g.stream = g.own_stream;
    g.owns_stream = 1;
    for (int i = 0; i < 2; i++) {
        if (cudaMallocHost(&g.stage[i], kStageBytes) != cudaSuccess) return 0;
        if (cudaEventCreateWithFlags(&g.stage_done[i], cudaEventDisableTiming) != cudaSuccess) return 0;
    }
    if (cudaEventCreate(&g.t0) != cudaSuccess || cudaEventCreate(&g.t1) != cudaSuccess) return 0;
    if (cudaMalloc((void **)&g.dev_status, 64) != cudaSuccess) return 0;
    if (cudaMemset(g.dev_status, 0, 64) != cudaSuccess) return 0;
    g.ready = 1;
    return 1;
}

int iris_dev_available(void) { return g.ready; }
const char *iris_dev_name(void) { return g.ready ? g.name : "none"; }

void iris_dev_cleanup(void) {
    if (!g.ready) return;
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
    sm100_release();
    if (g.scratch) cuda_ok(cudaFree(g.scratch), "free");
    g.scratch = NULL;
    g.scratch_bytes = 0;
    cuda_ok(cudaFree(g.dev_status), "free");
    g.dev_status = NULL;
    for (int i = 0; i < 2; i++) {
        cuda_ok(cudaFreeHost(g.stage[i]), "free host");
        cuda_ok(cudaEventDestroy(g.stage_done[i]), "event destroy");
    }
    cuda_ok(cudaEventDestroy(g.t0), "event destroy");
    cuda_ok(cudaEventDestroy(g.t1), "event destroy");
    cuda_ok(cudaStreamDestroy(g.own_stream), "stream destroy");
    g.ready = 0;
}

int iris_b200_attach_stream(void *cuda_stream) {
    if (!require_device("attach_stream")) return IRIS_B200_ENODEV;
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
    g.stream = cuda_stream ? (cudaStream_t)cuda_stream : g.own_stream;
    g.owns_stream = cuda_stream == NULL;
    return IRIS_B200_OK;
}

int iris_b200_use_stream(void *cuda_stream) {
    if (!require_device("use_stream")) return IRIS_B200_ENODEV;
    g.stream = cuda_stream ? (cudaStream_t)cuda_stream : g.own_stream;
    g.owns_stream = cuda_stream == NULL;
    return IRIS_B200_OK;
}

void *iris_b200_stream(void) { return g.ready ? (void *)g.stream : NULL; }

int iris_b200_timer_start(void) {
    if (!require_device("timer_start")) return IRIS_B200_ENODEV;
    return cuda_ok(cudaEventRecord(g.t0, g.stream), "event record") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

float iris_b200_timer_stop_ms(void) {
    if (!require_device("timer_stop")) return -1.0f;
    float ms = -1.0f;
    if (!cuda_ok(cudaEventRecord(g.t1, g.stream), "event record")) return -1.0f;
    if (!cuda_ok(cudaEventSynchronize(g.t1), "event sync")) return -1.0f;
    if (!cuda_ok(cudaEventElapsedTime(&ms, g.t0, g.t1), "event elapsed")) return -1.0f;
    return ms;
}

unsigned long long iris_b200_launch_count(void) { return g.launches; }

/* Numbered timing marks: events created on first use, recorded on the
 * library's stream. */
static const int kMaxMarks = 8192;
static cudaEvent_t g_marks[kMaxMarks];
static unsigned char g_mark_made[kMaxMarks];

int iris_b200_mark(int id) {
    if (!require_device("mark")) return IRIS_B200_ENODEV;
    if (id < 0 || id >= kMaxMarks) return IRIS_B200_EINVAL;
    if (!g_mark_made[id]) {
        if (!cuda_ok(cudaEventCreate(&g_marks[id]), "event create")) return IRIS_B200_ECUDA;
        g_mark_made[id] = 1;
    }
    return cuda_ok(cudaEventRecord(g_marks[id], g.stream), "event record") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}

float iris_b200_mark_elapsed_ms(int from, int to) {
    if (!require_device("mark_elapsed")) return -1.0f;
    if (from < 0 || to < 0 || from >= kMaxMarks || to >= kMaxMarks || !g_mark_made[from] || !g_mark_made[to])
        return -1.0f;
    float ms = -1.0f;
    if (!cuda_ok(cudaEventSynchronize(g_marks[to]), "event sync")) return -1.0f;
    if (!cuda_ok(cudaEventElapsedTime(&ms, g_marks[from], g_marks[to]), "event elapsed")) return -1.0f;
    return ms;
}

int iris_b200_check_device_status(void) {
    if (!require_device("check_device_status")) return IRIS_B200_ENODEV;
    unsigned int st[4] = {0, 0, 0, 0};
    if (!cuda_ok(cudaStreamSynchronize(g.stream), "sync")) return g.last_error;
    if (!cuda_ok(cudaMemcpy(st, g.dev_status, sizeof(st), cudaMemcpyDeviceToHost), "status read"))
        return g.last_error;
    if (st[0] != 0) {
        char msg[160];
        snprintf(msg, sizeof(msg), "wait timed out in kernel (site %u, block %u, aux %u)", st[1], st[2], st[3]);
        set_error(IRIS_B200_ETIMEOUT, "device wait", msg);
        cuda_ok(cudaMemset(g.dev_status, 0, 64), "status clear");
        /* A kernel that gave up may have left key-split tickets half used. */
        sm100_reset_split();
    }
    return g.last_error;
}

void *iris_dev_alloc(size_t bytes) {
    void *p = NULL;
    if (!g.ready) return NULL;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) {
        (void)cudaGetLastError();
        return NULL;
    }
    return p;
}

void iris_dev_free(void *p) {
    if (!p) return;
    /* Pending work may still use the buffer. */
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
    cuda_ok(cudaFree(p), "free");
}

/* Rows are packed into the pinned buffers by the CPU while the copy engine
 * drains the other buffer; a row wider than a buffer goes in pieces. */
void iris_dev_upload_2d(void *dst, size_t dst_stride, const void *src, size_t src_stride,
                        size_t row_bytes, size_t rows) {
    if (!require_device("upload") || row_bytes == 0 || rows == 0) return;
    size_t piece = row_bytes < kStageBytes ? row_bytes : kStageBytes;
    size_t rows_per_chunk = row_bytes <= kStageBytes ? kStageBytes / row_bytes : 1;
    int buf = 0;
    for (size_t r0 = 0; r0 < rows; r0 += rows_per_chunk) {
        size_t nr = rows - r0 < rows_per_chunk ? rows - r0 : rows_per_chunk;
        for (size_t off = 0; off < row_bytes; off += piece) {
            size_t len = row_bytes - off < piece ? row_bytes - off : piece;
            if (!cuda_ok(cudaEventSynchronize(g.stage_done[buf]), "event sync")) return;
            char *stage = (char *)g.stage[buf];
            if (src_stride == len && nr > 1 && off == 0 && row_bytes == len) {
                memcpy(stage, (const char *)src + r0 * src_stride, nr * len);
            } else {
                for (size_t r = 0; r < nr; r++)
                    memcpy(stage + r * len, (const char *)src + (r0 + r) * src_stride + off, len);
            }
            if (!cuda_ok(cudaMemcpy2DAsync((char *)dst + r0 * dst_stride + off, dst_stride, stage, len,
                                           len, nr, cudaMemcpyHostToDevice, g.stream), "upload"))
                return;
            cuda_ok(cudaEventRecord(g.stage_done[buf], g.stream), "event record");
            buf ^= 1;
        }
    }
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
}

/* Page-locked host memory is copied by the DMA engine directly; pageable
 * memory goes through the pinned staging buffers. */
static bool host_is_pinned(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

void iris_dev_upload(void *dst, const void *src, size_t bytes) {
    if (!bytes) return;
    if (g.ready && host_is_pinned(src)) {
        if (cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g.stream), "upload"))
            cuda_ok(cudaStreamSynchronize(g.stream), "sync");
        return;
    }
    iris_dev_upload_2d(dst, bytes, src, bytes, bytes, 1);
}

void iris_dev_download(void *dst, const void *src, size_t bytes) {
    if (!require_device("download") || bytes == 0) return;
    if (!cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g.stream), "download")) return;
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
}

void iris_dev_sync(void) {
    if (!g.ready) return;
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
}

void iris_dev_f32_to_bf16(uint16_t *dst, const float *src, size_t n) {
    if (!require_device("f32_to_bf16") || n == 0) return;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)g.sm_count * 16) blocks = (size_t)g.sm_count * 16;
    k_f32_to_bf16<<<(unsigned)blocks, 256, 0, g.stream>>>(dst, src, n);
    after_launch("f32_to_bf16");
}

}  // extern "C"
