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
    case IRIS_B200_EPROTO: return "ring ranks disagree";
    case IRIS_B200_ECHECK: return "self-check of the checking build failed";
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
    unsigned int st[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (!cuda_ok(cudaStreamSynchronize(g.stream), "sync")) return g.last_error;
    if (!cuda_ok(cudaMemcpy(st, g.dev_status, sizeof(st), cudaMemcpyDeviceToHost), "status read"))
        return g.last_error;
    if (st[4] != 0) {
        /* only the self-checking build (-DIRIS_B200_CHECK) writes these words */
        char msg[160];
        snprintf(msg, sizeof(msg), "self-check failed in kernel (site %u, block %u, aux %u)", st[5], st[6], st[7]);
        set_error(IRIS_B200_ECHECK, "device check", msg);
        if (st[0] == 0) cuda_ok(cudaMemset(g.dev_status, 0, 64), "status clear");
    }
    if (st[0] != 0) {
        char msg[160];
        snprintf(msg, sizeof(msg), "wait timed out in kernel (site %u, block %u, aux %u)", st[1], st[2], st[3]);
        set_error(IRIS_B200_ETIMEOUT, "device wait", msg);
        cuda_ok(cudaMemset(g.dev_status, 0, 64), "status clear");
        /* A kernel that gave up may have left key-split tickets and work-list
         * counters half used, and a ring call its peers out of step. */
        sm100_reset_split();
        ring_mark_failed();
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
    /* Kernels enqueued earlier may still read or write the buffer: the
     * reference's contract (iris_cuda.cu:181-186) is that free() is safe
     * right after the last launch that used it. */
    if (g.ready) cuda_ok(cudaStreamSynchronize(g.stream), "sync");
    cuda_ok(cudaFree(p), "free");
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

/* One tile of a pageable host matrix -> device through a pinned buffer:
 * `nrows` rows of `nbytes` starting at column byte `col`. The CPU packs the
 * tile while the copy engine still drains the other buffer. */
static bool stage_tile(int which, char *dst, size_t dst_stride, const char *src, size_t src_stride, size_t col,
                       size_t nbytes, size_t nrows) {
    if (!cuda_ok(cudaEventSynchronize(g.stage_done[which]), "event sync")) return false;
    char *pin = (char *)g.stage[which];
    if (src_stride == nbytes && col == 0) {
        memcpy(pin, src, nrows * nbytes);                   /* the rows are contiguous on the host */
    } else {
        for (size_t r = 0; r < nrows; r++) memcpy(pin + r * nbytes, src + r * src_stride + col, nbytes);
    }
    if (!cuda_ok(cudaMemcpy2DAsync(dst + col, dst_stride, pin, nbytes, nbytes, nrows, cudaMemcpyHostToDevice, g.stream),
                 "upload"))
        return false;
    return cuda_ok(cudaEventRecord(g.stage_done[which], g.stream), "event record");
}

/* Blocking strided upload (iris_dev.h: iris_dev_upload_2d). Pinned sources
 * are one 2-D DMA; pageable ones are cut into tiles that fit a staging
 * buffer (whole rows when a row fits, else column pieces of single rows). */
void iris_dev_upload_2d(void *dst, size_t dst_stride, const void *src, size_t src_stride,
                        size_t row_bytes, size_t rows) {
    if (!require_device("upload") || row_bytes == 0 || rows == 0) return;
    if (host_is_pinned(src)) {
        if (cuda_ok(cudaMemcpy2DAsync(dst, dst_stride, src, src_stride, row_bytes, rows, cudaMemcpyHostToDevice,
                                      g.stream), "upload"))
            cuda_ok(cudaStreamSynchronize(g.stream), "sync");
        return;
    }
    const size_t tile_cols = row_bytes < kStageBytes ? row_bytes : kStageBytes;
    const size_t tile_rows = kStageBytes / tile_cols;         /* >= 1 */
    int which = 0;
    bool ok = true;
    for (size_t r = 0; r < rows && ok; r += tile_rows) {
        const size_t nrows = rows - r < tile_rows ? rows - r : tile_rows;
        for (size_t col = 0; col < row_bytes && ok; col += tile_cols, which ^= 1) {
            const size_t nbytes = row_bytes - col < tile_cols ? row_bytes - col : tile_cols;
            ok = stage_tile(which, (char *)dst + r * dst_stride, dst_stride, (const char *)src + r * src_stride,
                            src_stride, col, nbytes, nrows);
        }
    }
    cuda_ok(cudaStreamSynchronize(g.stream), "sync");
}

void iris_dev_upload(void *dst, const void *src, size_t bytes) {
    if (!bytes) return;
    iris_dev_upload_2d(dst, bytes, src, bytes, bytes, 1);
}

/* Stream-ordered copies between page-locked host memory and the device, on a
 * stream of the caller's (NULL: the library's): they return at once, and the
 * caller orders them against the operations with events or by sharing the
 * stream. With three buffer sets this is what overlaps the upload of step
 * i + 1 and the download of step i - 1 with the kernels of step i. */
int iris_b200_upload_async(void *dst, const void *src, size_t bytes, void *cuda_stream) {
    if (!require_device("upload_async")) return IRIS_B200_ENODEV;
    if (!bytes) return IRIS_B200_OK;
    if (!dst || !src || !host_is_pinned(src)) {
        set_error(IRIS_B200_EINVAL, "upload_async", "source must be page-locked host memory");
        return IRIS_B200_EINVAL;
    }
    cudaStream_t st = cuda_stream ? (cudaStream_t)cuda_stream : g.stream;
    return cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st), "upload_async") ? IRIS_B200_OK
                                                                                                 : IRIS_B200_ECUDA;
}

int iris_b200_download_async(void *dst, const void *src, size_t bytes, void *cuda_stream) {
    if (!require_device("download_async")) return IRIS_B200_ENODEV;
    if (!bytes) return IRIS_B200_OK;
    if (!dst || !src || !host_is_pinned(dst)) {
        set_error(IRIS_B200_EINVAL, "download_async", "destination must be page-locked host memory");
        return IRIS_B200_EINVAL;
    }
    cudaStream_t st = cuda_stream ? (cudaStream_t)cuda_stream : g.stream;
    return cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, st), "download_async") ? IRIS_B200_OK
                                                                                                   : IRIS_B200_ECUDA;
}

/* Page-locked host memory for the asynchronous copies. */
void *iris_b200_host_alloc(size_t bytes) {
    void *p = NULL;
    if (!g.ready) return NULL;
    if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) {
        (void)cudaGetLastError();
        return NULL;
    }
    return p;
}
void iris_b200_host_free(void *p) {
    if (p) cuda_ok(cudaFreeHost(p), "free host");
}

/* Streams and events for callers that have no CUDA headers of their own
 * (plain-C hosts): what the pipelined copies above are ordered with. */
void *iris_b200_stream_create(void) {
    cudaStream_t st = NULL;
    if (!g.ready || !cuda_ok(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "stream create")) return NULL;
    return (void *)st;
}
void iris_b200_stream_destroy(void *cuda_stream) {
    if (cuda_stream) cuda_ok(cudaStreamDestroy((cudaStream_t)cuda_stream), "stream destroy");
}
void *iris_b200_event_create(void) {
    cudaEvent_t ev = NULL;
    if (!g.ready || !cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "event create")) return NULL;
    return (void *)ev;
}
void iris_b200_event_destroy(void *event) {
    if (event) cuda_ok(cudaEventDestroy((cudaEvent_t)event), "event destroy");
}
/* record: NULL stream = the library's. wait: the stream waits for the event. */
int iris_b200_event_record(void *event, void *cuda_stream) {
    if (!require_device("event_record") || !event) return IRIS_B200_EINVAL;
    return cuda_ok(cudaEventRecord((cudaEvent_t)event, cuda_stream ? (cudaStream_t)cuda_stream : g.stream), "event record")
               ? IRIS_B200_OK : IRIS_B200_ECUDA;
}
int iris_b200_stream_wait_event(void *cuda_stream, void *event) {
    if (!require_device("stream_wait_event") || !event) return IRIS_B200_EINVAL;
    return cuda_ok(cudaStreamWaitEvent(cuda_stream ? (cudaStream_t)cuda_stream : g.stream, (cudaEvent_t)event, 0),
                   "stream wait") ? IRIS_B200_OK : IRIS_B200_ECUDA;
}
int iris_b200_stream_sync(void *cuda_stream) {
    if (!require_device("stream_sync")) return IRIS_B200_ENODEV;
    return cuda_ok(cudaStreamSynchronize(cuda_stream ? (cudaStream_t)cuda_stream : g.stream), "sync") ? IRIS_B200_OK
                                                                                                      : IRIS_B200_ECUDA;
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
