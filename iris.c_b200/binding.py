"""ctypes declarations of every entry point in include/*.h."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libiris_b200.so")

VP, INT, FLT, SZ, U64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_ulonglong


class IrisB200Error(RuntimeError):
    pass


# name -> (restype, argtypes); one entry per declaration in include/*.h
SIGNATURES = {
    # iris_dev.h
    "iris_dev_init": (INT, []),
    "iris_dev_available": (INT, []),
    "iris_dev_name": (C.c_char_p, []),
    "iris_dev_cleanup": (None, []),
    "iris_dev_alloc": (VP, [SZ]),
    "iris_dev_free": (None, [VP]),
    "iris_dev_upload": (None, [VP, VP, SZ]),
    "iris_dev_download": (None, [VP, VP, SZ]),
    "iris_dev_upload_2d": (None, [VP, SZ, VP, SZ, SZ, SZ]),
    "iris_dev_sync": (None, []),
    "iris_dev_f32_to_bf16": (None, [VP, VP, SZ]),
    "iris_dev_linear_bf16": (None, [VP, VP, VP, INT, INT, INT]),
    "iris_dev_linear_f32": (None, [VP, VP, VP, INT, INT, INT]),
    "iris_dev_layer_norm_mod": (None, [VP, VP, VP, VP, INT, INT, FLT]),
    "iris_dev_rms_norm": (None, [VP, VP, VP, INT, INT, FLT]),
    "iris_dev_rms_norm_mod": (None, [VP, VP, VP, VP, INT, INT, FLT]),
    "iris_dev_rms_norm_residual": (None, [VP, VP, VP, VP, INT, INT, FLT]),
    "iris_dev_swiglu": (None, [VP, INT, VP, VP, INT, INT, INT]),
    "iris_dev_residual": (None, [VP, VP, VP, INT, INT]),
    "iris_dev_head_norm_rope": (None, [VP, INT, VP, VP, VP, INT, INT, INT, FLT, INT]),
    "iris_dev_attention": (None, [VP, INT, VP, VP, VP, INT, INT, INT, INT, INT, INT, FLT, INT, VP]),
    # iris_kernels.h
    "iris_softmax": (None, [VP, INT, INT]),
    "iris_attention": (None, [VP, VP, VP, VP, INT, INT, INT, INT, INT, FLT]),
    "iris_flash_attention": (None, [VP, VP, VP, VP, INT, INT, INT, INT, FLT]),
    "iris_apply_rope": (None, [VP, VP, INT, INT, INT, INT]),
    "iris_compute_rope_freqs": (None, [VP, VP, INT, INT, FLT]),
    "iris_softmax_cpu": (None, [VP, INT, INT]),
    # iris_b200.h
    "iris_b200_last_error": (INT, []),
    "iris_b200_clear_error": (None, []),
    "iris_b200_strerror": (C.c_char_p, [INT]),
    "iris_b200_check_device_status": (INT, []),
    "iris_b200_set_device": (INT, [INT]),
    "iris_b200_attach_stream": (INT, [VP]),
    "iris_b200_use_stream": (INT, [VP]),
    "iris_b200_stream": (VP, []),
    "iris_b200_timer_start": (INT, []),
    "iris_b200_timer_stop_ms": (FLT, []),
    "iris_b200_launch_count": (U64, []),
    "iris_b200_mark": (INT, [INT]),
    "iris_b200_mark_elapsed_ms": (FLT, [INT, INT]),
    "iris_b200_qk_norm_rope": (INT, [VP, VP, INT, VP, VP, VP, VP, INT, INT, INT, FLT, INT]),
    "iris_b200_linear_qk_norm_rope": (INT, [VP, INT, VP, VP, INT, INT, INT, INT, VP, VP, VP, VP, FLT]),
    "iris_b200_linear_cta_pairs": (INT, [INT]),
    "iris_b200_linear_plan": (INT, [INT, INT, INT, INT, INT, INT, VP, VP, VP, VP, INT]),
    "iris_b200_linear_glu": (INT, [VP, INT, VP, INT, VP, VP, INT, INT, INT, INT, VP, VP, VP, VP, FLT]),
    "iris_b200_linear_residual": (INT, [VP, INT, VP, INT, VP, INT, VP, INT, INT, INT]),
    "iris_b200_single_block_scratch_bytes": (SZ, [INT, INT, INT]),
    "iris_b200_single_block": (INT, [VP, VP, VP, VP, VP, VP, VP, VP, VP, INT, INT, INT, INT, VP]),
    "iris_b200_single_block_segments": (INT, [VP, VP, VP, VP, VP, VP, VP, INT, VP, VP, INT, INT, INT, INT, FLT, VP]),
    "iris_b200_zimage_block_scratch_bytes": (SZ, [INT, INT, INT]),
    "iris_b200_zimage_block": (INT, [VP, VP, VP, VP, VP, VP, INT, INT, INT, INT, VP]),
    "iris_b200_single_block_tp_scratch_bytes": (SZ, [INT, INT, INT]),
    "iris_b200_single_block_tp": (INT, [VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, INT, INT, INT, VP]),
    "iris_b200_double_block_scratch_bytes": (SZ, [INT, INT, INT]),
    "iris_b200_double_block": (INT, [VP, VP, VP, VP, VP, VP, INT, INT, INT, INT, INT, VP]),
    "iris_b200_attention_ex": (INT, [VP, INT, VP, VP, VP, INT, INT, INT, INT, INT, INT, FLT, INT, VP, INT]),
    "iris_b200_attention_kernel_for": (INT, [VP, INT, VP, VP, VP, INT, INT, INT, INT, INT]),
    "iris_b200_head_shard": (INT, [INT, INT, INT, C.POINTER(INT), C.POINTER(INT)]),
    "iris_b200_cfg_shard": (INT, [INT, INT, INT, INT, C.POINTER(INT), C.POINTER(INT), C.POINTER(INT), C.POINTER(INT)]),
    "iris_b200_seq_shard": (INT, [INT, INT, INT, C.POINTER(INT), C.POINTER(INT)]),
    "iris_b200_ring_source": (INT, [INT, INT, INT]),
    "iris_b200_ring_plan": (INT, [INT, INT, VP, VP]),
    "iris_b200_attention_chunk": (INT, [VP, INT, VP, INT, VP, VP, INT, INT, INT, INT, FLT, VP, VP, VP, INT, INT]),
    "iris_b200_ring_unique_id": (INT, [VP]),
    "iris_b200_ring_init": (INT, [INT, INT, VP]),
    "iris_b200_ring_attention": (INT, [VP, INT, VP, VP, VP, INT, VP, INT, FLT]),
    "iris_b200_ring_destroy": (None, []),
    "iris_b200_attention_noalloc": (INT, [VP, INT, VP, VP, VP, INT, INT, INT, INT, FLT, INT]),
    "iris_b200_attention_noalloc_max_elems": (SZ, []),
    "iris_b200_attention_runs": (INT, [VP, INT, VP, INT, INT, INT, FLT, VP, VP, INT, VP, VP, INT, VP, INT, VP,
                                       C.c_uint32, INT]),
    "iris_b200_attention_runs_plan": (INT, [VP, INT, INT, INT, INT, INT, VP, VP]),
    "iris_b200_ring_launch_plan": (INT, [INT, INT, VP, INT, INT, INT, VP, VP, VP]),
    "iris_b200_set_wait_limit_us": (INT, [C.c_uint]),
    "iris_b200_inject_fault": (INT, [INT]),
    "iris_b200_upload_async": (INT, [VP, VP, SZ, VP]),
    "iris_b200_download_async": (INT, [VP, VP, SZ, VP]),
    "iris_b200_host_alloc": (VP, [SZ]),
    "iris_b200_host_free": (None, [VP]),
    "iris_b200_stream_create": (VP, []),
    "iris_b200_stream_destroy": (None, [VP]),
    "iris_b200_event_create": (VP, []),
    "iris_b200_event_destroy": (None, [VP]),
    "iris_b200_event_record": (INT, [VP, VP]),
    "iris_b200_stream_wait_event": (INT, [VP, VP]),
    "iris_b200_stream_sync": (INT, [VP]),
    "iris_b200_ring_configure": (INT, [INT, INT]),
    "iris_b200_ring_transport": (INT, []),
    "iris_b200_outproj_residual": (INT, [VP, VP, INT, VP, INT, VP, VP, INT, INT]),
    "iris_b200_ring_loopback": (INT, [INT, VP, INT, INT, C.c_uint, VP, INT, VP, VP, VP]),
    "iris_b200_ring_loopback_digest": (C.c_uint64, [INT, VP, INT, INT, INT]),
    "iris_b200_ring_trace": (INT, [INT]),
    "iris_b200_ring_timeline": (INT, [VP, INT]),
}

KERNEL_AUTO, KERNEL_TCGEN05, KERNEL_GENERIC = 0, 1, 2


class LoopFault(C.Structure):
    """iris_b200_loop_fault of include/iris_b200.h."""
    _fields_ = [("kind", INT), ("rank", INT), ("call", INT), ("step", INT), ("delay_us", C.c_uint)]


class Segment(C.Structure):
    """iris_b200_segment of include/iris_b200.h."""
    _fields_ = [("start", INT), ("len", INT), ("mod", VP)]


class ZImageWeights(C.Structure):
    """iris_b200_zimage_weights of include/iris_b200.h."""
    _fields_ = [(n, VP) for n in ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k", "attn_norm1", "attn_norm2",
                                  "ffn_norm1", "ffn_norm2")]


class StreamWeights(C.Structure):
    """iris_b200_stream_weights of include/iris_b200.h."""
    _fields_ = [(n, VP) for n in ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k", "mod")]


class KeyRun(C.Structure):
    """iris_b200_key_run of include/iris_b200.h."""
    _fields_ = [("view", INT), ("row0", INT), ("rows", INT), ("arrive", INT), ("rows_per_word", INT)]


class Lib:
    """The loaded library with typed entry points as attributes."""

    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise IrisB200Error(
                "%s not found: build it with `make -C iris.c_b200` (nvcc, sm_100a); "
                "there is no fallback implementation" % path)
        self.path = path
        self.cdll = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.cdll, name)       # AttributeError = symbol missing
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)

    # -- small conveniences over the raw ABI (host numpy <-> device pointers) --

    def init(self, device=None):
        if device is not None and not self.iris_dev_available():
            self.iris_b200_set_device(int(device))
        if not self.iris_dev_init():
            raise IrisB200Error("iris_dev_init failed: no usable sm_100 GPU")

    def check(self):
        code = self.iris_b200_check_device_status()
        if code:
            msg = self.iris_b200_strerror(code).decode()
            self.iris_b200_clear_error()
            raise IrisB200Error("iris_b200 error %d: %s" % (code, msg))

    def alloc(self, nbytes):
        p = self.iris_dev_alloc(nbytes)
        if not p:
            raise IrisB200Error("iris_dev_alloc(%d) failed" % nbytes)
        return p

    def to_device(self, arr):
        import numpy as np
        arr = np.ascontiguousarray(arr)
        p = self.alloc(arr.nbytes)
        self.iris_dev_upload(p, arr.ctypes.data, arr.nbytes)
        return p

    def to_host(self, ptr, shape, dtype):
        import numpy as np
        out = np.empty(shape, dtype)
        self.iris_dev_download(out.ctypes.data, ptr, out.nbytes)
        return out


_lib = None


def load():
    global _lib
    if _lib is None:
        _lib = Lib()
    return _lib
