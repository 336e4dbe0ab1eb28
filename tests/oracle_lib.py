"""ctypes access to the CPU checkers used by the tests.

* ``oracle()``  -> ``oracle/liboracle.so``, the CPU restatement of the path.
* ``ref(kind)`` -> ``oracle/_ref/libiris_ref_{generic,blas}.so``, the
  reference's own CPU code compiled from its sources (None when absent).

Test infrastructure only: the shipped library never loads these.
"""
import ctypes as C
import functools
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
INT, FLT, SZ = C.c_int, C.c_float, C.c_size_t


class _OptPtr:
    """ndpointer that also accepts None (NULL)."""

    def __init__(self, base):
        self.base = base

    def from_param(self, obj):
        if obj is None:
            return C.c_void_p(0)
        return self.base.from_param(obj)


i32p_opt = _OptPtr(i32p)
f32p_opt = _OptPtr(f32p)


def _sig(lib, name, argtypes, restype=None):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


@functools.lru_cache(None)
def oracle():
    path = os.path.join(ORACLE_DIR, "liboracle.so")
    if not os.path.exists(path):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "liboracle.so"])
    lib = C.CDLL(path)
    _sig(lib, "orc_rng_seed", [C.c_uint64])
    _sig(lib, "orc_random_uniform", [], FLT)
    _sig(lib, "orc_randn", [f32p, SZ])
    _sig(lib, "orc_f32_to_bf16", [u16p, f32p, SZ])
    _sig(lib, "orc_bf16_to_f32", [f32p, u16p, SZ])
    _sig(lib, "orc_round_bf16", [f32p, SZ])
    _sig(lib, "orc_fast_expf", [FLT], FLT)
    _sig(lib, "orc_softmax", [f32p, INT, INT])
    _sig(lib, "orc_attention", [f32p, f32p, f32p, f32p, INT, INT, INT, INT, INT, FLT])
    _sig(lib, "orc_flash_attention", [f32p, f32p, f32p, f32p, INT, INT, INT, INT, FLT])
    _sig(lib, "orc_apply_rope", [f32p, f32p, INT, INT, INT, INT])
    _sig(lib, "orc_compute_rope_freqs", [f32p, i32p, INT, INT, FLT])
    _sig(lib, "orc_head_norm_rope_f32", [C.c_void_p, INT, f32p, f32p, f32p, INT, INT, INT, FLT, INT])
    _sig(lib, "orc_head_norm_rope_bf16", [C.c_void_p, INT, f32p, f32p, f32p, INT, INT, INT, FLT, INT])
    _sig(lib, "orc_dev_attention", [C.c_void_p, INT, C.c_void_p, C.c_void_p, C.c_void_p, INT, INT, INT,
                                    INT, INT, INT, FLT, INT, i32p_opt, i32p_opt, INT, INT])
    _sig(lib, "orc_flux_rope_text", [f32p, f32p, INT, INT, FLT])
    _sig(lib, "orc_flux_rope_image", [f32p, f32p, INT, INT, INT, FLT, INT])
    _sig(lib, "orc_f3_joint_rope", [f32p, f32p, INT, INT, INT, i32p, i32p, INT, INT, FLT], INT)
    _sig(lib, "orc_zi_rope", [f32p, f32p, i32p, INT, FLT])
    _sig(lib, "orc_zi_positions", [i32p, i32p, INT, INT, INT], INT)
    _sig(lib, "orc_layer_norm_mod", [u16p, f32p, f32p_opt, f32p_opt, INT, INT, FLT])
    _sig(lib, "orc_swiglu", [C.c_void_p, INT, C.c_void_p, C.c_void_p, INT, INT, INT])
    _sig(lib, "orc_residual", [f32p, f32p, f32p_opt, INT, INT])
    _sig(lib, "orc_linear", [f32p, INT, u16p, INT, u16p, INT, INT, INT, INT, INT])
    _sig(lib, "orc_single_block", [f32p, u16p, u16p, f32p, f32p, f32p, f32p, f32p, INT, INT, INT, INT,
                                   i32p_opt, INT], INT)
    _sig(lib, "orc_rms_norm_mod", [u16p, f32p, f32p, f32p_opt, INT, INT, FLT])
    _sig(lib, "orc_rms_norm_residual", [f32p, f32p, f32p, f32p_opt, INT, INT, FLT])
    _sig(lib, "orc_compare_heads", [C.c_void_p, INT, C.c_void_p, INT, INT, INT, INT, i32p_opt, INT, f32p, f32p])
    return lib


@functools.lru_cache(None)
def ref(kind="generic"):
    path = os.path.join(ORACLE_DIR, "_ref", "libiris_ref_%s.so" % kind)
    if not os.path.exists(path):
        return None
    try:
        lib = C.CDLL(path)
    except OSError:
        return None
    _sig(lib, "iris_rng_seed", [C.c_uint64])
    _sig(lib, "iris_random_uniform", [], FLT)
    _sig(lib, "iris_randn", [f32p, INT])
    _sig(lib, "iris_softmax", [f32p, INT, INT])
    _sig(lib, "iris_attention", [f32p, f32p, f32p, f32p, INT, INT, INT, INT, INT, FLT])
    _sig(lib, "iris_flash_attention", [f32p, f32p, f32p, f32p, INT, INT, INT, INT, FLT])
    _sig(lib, "iris_apply_rope", [f32p, f32p, INT, INT, INT, INT])
    _sig(lib, "iris_compute_rope_freqs", [f32p, i32p, INT, INT, FLT])
    _sig(lib, "ref_flux_qk_norm", [f32p, f32p, f32p, f32p, INT, INT, INT, FLT])
    _sig(lib, "ref_flux_rope_text", [f32p, f32p, INT, INT, FLT])
    _sig(lib, "ref_flux_rope_2d", [f32p, f32p, INT, INT, INT, FLT])
    _sig(lib, "ref_flux_rope_2d_t", [f32p, f32p, INT, INT, INT, FLT, INT])
    _sig(lib, "ref_flux_apply_rope_2d", [f32p, f32p, f32p, INT, INT, INT])
    _sig(lib, "ref_flux_joint_attention", [f32p] * 8 + [INT] * 4, INT)
    _sig(lib, "ref_flux_mha", [f32p] * 4 + [INT] * 3, INT)
    _sig(lib, "ref_flux_attn_threads", [INT], INT)
    _sig(lib, "ref_flux_single_block", [f32p] * 11 + [INT] * 5, INT)
    _sig(lib, "ref_flux_double_block", [f32p, f32p, C.c_void_p, C.c_void_p] + [f32p] * 6 + [INT] * 5, INT)
    _sig(lib, "ref_f3_head_rms_norm", [f32p, f32p, INT, INT, INT, FLT])
    _sig(lib, "ref_f3_apply_rope", [f32p, f32p, f32p, INT, INT, INT])
    _sig(lib, "ref_f3_joint_rope", [f32p, f32p, INT, INT, INT, i32p, i32p, INT, INT, INT, FLT], INT)
    _sig(lib, "ref_f3_attention", [f32p] * 4 + [INT] * 3, INT)
    _sig(lib, "ref_f3_block", [f32p, C.c_void_p, f32p, f32p, i32p, i32p, C.c_void_p, INT, f32p, f32p, INT, INT, INT, INT, FLT], INT)
    _sig(lib, "ref_zi_qk_norm", [f32p, f32p, INT, INT, INT, FLT])
    _sig(lib, "ref_zi_apply_rope", [f32p, i32p, INT, INT, INT])
    _sig(lib, "ref_zi_block", [f32p, C.c_void_p, f32p, f32p, f32p_opt, i32p, i32p_opt, INT, INT, INT, INT], INT)
    _sig(lib, "ref_zi_attention_identity", [f32p, f32p, i32p, i32p_opt, INT, INT, INT], INT)
    if kind == "blas":
        _sig(lib, "openblas_set_num_threads", [INT])
    return lib


@functools.lru_cache(None)
def ref_cuda():
    """The reference's own CUDA backend (iris_cuda.cu compiled unmodified for
    sm_100), or None when it was not built or cannot load."""
    path = os.path.join(ORACLE_DIR, "_ref", "libiris_ref_cuda.so")
    if not os.path.exists(path):
        return None
    try:
        lib = C.CDLL(path)
    except OSError:
        return None
    VP = C.c_void_p
    _sig(lib, "iris_dev_init", [], INT)
    _sig(lib, "iris_dev_sync", [])
    _sig(lib, "iris_dev_name", [], C.c_char_p)
    _sig(lib, "iris_dev_head_norm_rope", [VP, INT, VP, VP, VP, INT, INT, INT, FLT, INT])
    _sig(lib, "iris_dev_attention", [VP, INT, VP, VP, VP, INT, INT, INT, INT, INT, INT, FLT, INT, VP])
    _sig(lib, "iris_dev_linear_bf16", [VP, VP, VP, INT, INT, INT])
    _sig(lib, "iris_dev_linear_f32", [VP, VP, VP, INT, INT, INT])
    _sig(lib, "iris_dev_layer_norm_mod", [VP, VP, VP, VP, INT, INT, FLT])
    _sig(lib, "iris_dev_swiglu", [VP, INT, VP, VP, INT, INT, INT])
    _sig(lib, "iris_dev_residual", [VP, VP, VP, INT, INT])
    _sig(lib, "iris_dev_rms_norm_mod", [VP, VP, VP, VP, INT, INT, FLT])
    _sig(lib, "iris_dev_rms_norm_residual", [VP, VP, VP, VP, INT, INT, FLT])
    return lib


# ---------------------------------------------------------------------------
# numpy-level helpers shared by the tests
# ---------------------------------------------------------------------------

def randn(seed, *shape):
    """N(0,1) fp32 from the reference's generator (iris_kernels.c:70-98)."""
    o = oracle()
    out = np.empty(shape, np.float32)
    o.orc_rng_seed(seed)
    o.orc_randn(out.reshape(-1), out.size)
    return out


def to_bf16(x):
    o = oracle()
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    o.orc_f32_to_bf16(out.reshape(-1), x.reshape(-1), x.size)
    return out


def from_bf16(x):
    o = oracle()
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    o.orc_bf16_to_f32(out.reshape(-1), x.reshape(-1), x.size)
    return out


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def dev_attention(q, k, v, heads, kv_heads=None, head_dim=128, scale=None, causal=0,
                  key_mask=None, rows=None, nthreads=0):
    """orc_dev_attention on contiguous fp32 [seq, heads*hd] arrays."""
    o = oracle()
    kv_heads = kv_heads or heads
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    seq_q, seq_k = q.shape[0], k.shape[0]
    assert k.shape[1] == v.shape[1]
    # q/k/v share one row stride in the device API: pad the narrower to the wider.
    ldi = max(q.shape[1], k.shape[1])
    if q.shape[1] != ldi:
        q = np.ascontiguousarray(np.pad(q, ((0, 0), (0, ldi - q.shape[1]))))
    if k.shape[1] != ldi:
        k = np.ascontiguousarray(np.pad(k, ((0, 0), (0, ldi - k.shape[1]))))
        v = np.ascontiguousarray(np.pad(v, ((0, 0), (0, ldi - v.shape[1]))))
    out = np.zeros((seq_q, heads * head_dim), np.float32)
    scale = scale if scale is not None else 1.0 / np.sqrt(head_dim)
    if key_mask is not None:
        key_mask = np.ascontiguousarray(key_mask, np.int32)
    nrows = 0
    if rows is not None:
        rows = np.ascontiguousarray(rows, np.int32)
        nrows = rows.size
    o.orc_dev_attention(_ptr(out), out.shape[1], _ptr(q), _ptr(k), _ptr(v), ldi, seq_q, seq_k,
                        heads, kv_heads, head_dim, scale, causal, key_mask, rows, nrows, nthreads)
    return out


def compare_heads(a, b, heads, head_dim=128, rows=None):
    """(max_abs[heads], cosine[heads]) between two fp32 [seq, heads*hd] arrays."""
    o = oracle()
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    mx = np.empty(heads, np.float32)
    cs = np.empty(heads, np.float32)
    nrows = 0
    if rows is not None:
        rows = np.ascontiguousarray(rows, np.int32)
        nrows = rows.size
    o.orc_compare_heads(_ptr(a), a.shape[1], _ptr(b), b.shape[1], a.shape[0], heads, head_dim,
                        rows, nrows, mx, cs)
    return mx, cs
