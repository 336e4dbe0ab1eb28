"""Inputs of one FLUX.2 single-stream block, shared by the CPU and GPU tests.

Seeded synthetic tensors with the model's shapes: hidden state N(0, 1),
weights N(0, 1 / in) rounded to bf16 (the checkpoints store bf16), per-head
norm weights near 1, a timestep embedding and an AdaLN weight from which the
modulation (shift | scale | gate) follows as in the reference
(iris_transformer_flux.c:3361-3385): mod = adaln . silu(t_emb).
"""
import numpy as np

import oracle_lib as ol
import path_cases as pc

D = 128

# klein4b widths on a short sequence, and a small case the CPU reference runs in seconds
SMALL = dict(name="flux2-block-small", family="flux2", heads=2, mlp=768, txt=32, img=(8, 8), refs=[], eps=1e-6)
MID = dict(name="flux2-block-mid", family="flux2", heads=4, mlp=1536, txt=40, img=(12, 11), refs=[], eps=1e-6)
ODD_HEADS = dict(name="flux2-block-3-heads", family="flux2", heads=3, mlp=1152, txt=40, img=(12, 11), refs=[], eps=1e-6)
KLEIN4B_SHORT = dict(name="klein4b-block-short", family="flux2", heads=24, mlp=9216, txt=64, img=(8, 16),
                     refs=[], eps=1e-6)
KLEIN4B = dict(name="klein4b-block-1024", family="flux2", heads=24, mlp=9216, txt=512, img=(64, 64), refs=[],
               eps=1e-6)


def block_inputs(case, seed=7):
    H, mlp = case["heads"], case["mlp"]
    dim, seq = H * D, pc.seq_len(case)
    ldh, ldc = 3 * dim + 2 * mlp, dim + mlp
    x = ol.randn(seed, seq, dim)
    w_in = ol.to_bf16(ol.randn(seed + 1, ldh, dim) / np.float32(np.sqrt(dim)))
    w_out = ol.to_bf16(ol.randn(seed + 2, dim, ldc) / np.float32(np.sqrt(ldc)))
    norm_q = (1.0 + 0.1 * ol.randn(seed + 3, D)).astype(np.float32)
    norm_k = (1.0 + 0.1 * ol.randn(seed + 4, D)).astype(np.float32)
    t_emb = ol.randn(seed + 5, dim)
    adaln = (ol.randn(seed + 6, 3 * dim, dim) * np.float32(0.5 / np.sqrt(dim))).astype(np.float32)
    silu = (t_emb / (1.0 + np.exp(-t_emb))).astype(np.float32)
    mod = (adaln.astype(np.float64) @ silu.astype(np.float64)).astype(np.float32)
    cos, sin, _ = pc.rope_tables(case)
    return dict(x=x, w_in=w_in, w_out=w_out, norm_q=norm_q, norm_k=norm_k, t_emb=t_emb, adaln=adaln, mod=mod,
                cos=cos, sin=sin, seq=seq, dim=dim, heads=H, mlp=mlp)


def oracle_block(inp, key_mask=None, nthreads=0):
    """x after the block, by the CPU restatement of the device sequence."""
    x = inp["x"].copy()
    rc = ol.oracle().orc_single_block(x, inp["w_in"], inp["w_out"], inp["norm_q"], inp["norm_k"], inp["mod"],
                                      inp["cos"], inp["sin"], inp["seq"], inp["dim"], inp["heads"], inp["mlp"],
                                      key_mask, nthreads)
    assert rc == 0
    return x


def delta_metrics(got, want, x0):
    """The block adds gate * projection to x: compare what was added.
    Returns (max |difference| / max |added|, cosine of the added parts)."""
    a = (got - x0).astype(np.float64).ravel()
    b = (want - x0).astype(np.float64).ravel()
    scale = np.abs(b).max()
    return np.abs(a - b).max() / scale, float(a @ b / np.sqrt((a @ a) * (b @ b)))


# ---------------------------------------------------------------------------
# double-stream block
# ---------------------------------------------------------------------------

import ctypes as C  # noqa: E402


class StreamWeights(C.Structure):
    """iris_b200_stream_weights of include/iris_b200.h; orc_stream_weights of
    oracle/iris_oracle.h has the same layout."""
    _fields_ = [(n, C.c_void_p) for n in ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k", "mod")]


STREAM_KEYS = ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k", "mod")


def stream_inputs(dim, mlp, seed):
    s = np.float32
    return dict(
        qkv=ol.to_bf16(ol.randn(seed, 3 * dim, dim) / s(np.sqrt(dim))),
        proj=ol.to_bf16(ol.randn(seed + 1, dim, dim) / s(np.sqrt(dim))),
        ff_in=ol.to_bf16(ol.randn(seed + 2, 2 * mlp, dim) / s(np.sqrt(dim))),
        ff_out=ol.to_bf16(ol.randn(seed + 3, dim, mlp) / s(np.sqrt(mlp))),
        norm_q=(1.0 + 0.1 * ol.randn(seed + 4, D)).astype(s),
        norm_k=(1.0 + 0.1 * ol.randn(seed + 5, D)).astype(s),
        mod=(0.4 * ol.randn(seed + 6, 6 * dim)).astype(s))


def double_inputs(case, seed=11):
    H, mlp = case["heads"], case["mlp"]
    dim, seq = H * D, pc.seq_len(case)
    cos, sin, _ = pc.rope_tables(case)
    return dict(x=ol.randn(seed, seq, dim), txt=stream_inputs(dim, mlp, seed + 10), img=stream_inputs(dim, mlp, seed + 20),
                cos=cos, sin=sin, seq=seq, txt_seq=case["txt"], dim=dim, heads=H, mlp=mlp)


def host_stream(st):
    """StreamWeights over host arrays (for the oracle)."""
    return StreamWeights(*[st[k].ctypes.data for k in STREAM_KEYS])


def oracle_double_block(inp, key_mask=None, nthreads=0):
    x = inp["x"].copy()
    o = ol.oracle()
    fn = o.orc_double_block
    fn.restype = C.c_int
    fn.argtypes = [ol.f32p, C.POINTER(StreamWeights), C.POINTER(StreamWeights), ol.f32p, ol.f32p] + [C.c_int] * 5 + \
                  [ol.i32p_opt, C.c_int]
    t, i = host_stream(inp["txt"]), host_stream(inp["img"])
    rc = fn(x, C.byref(t), C.byref(i), inp["cos"], inp["sin"], inp["seq"], inp["txt_seq"], inp["dim"], inp["heads"],
            inp["mlp"], key_mask, nthreads)
    assert rc == 0
    return x


# ---------------------------------------------------------------------------
# FLUX.3 block: the single-stream layout with the rows in segments (text,
# image, reference images), each with its own modulation
# ---------------------------------------------------------------------------

F3_SMALL = dict(name="flux3-block-small", family="flux3", heads=2, mlp=768, txt=33, img=(10, 10), refs=[(6, 6), (5, 7)],
                eps=1e-6)
F3_MID = dict(name="flux3-block-mid", family="flux3", heads=4, mlp=1536, txt=40, img=(12, 11), refs=[(8, 8)], eps=1e-6)
F3_KLEIN_SHORT = dict(name="flux3-block-24-heads", family="flux3", heads=24, mlp=9216, txt=64, img=(8, 12), refs=[(4, 8)],
                      eps=1e-6)


class Segment(C.Structure):
    """iris_b200_segment of include/iris_b200.h."""
    _fields_ = [("start", C.c_int), ("len", C.c_int), ("mod", C.c_void_p)]


def f3_inputs(case, seed=51):
    inp = block_inputs(case, seed)
    dim, txt = inp["dim"], case["txt"]
    img = case["img"][0] * case["img"][1]
    cond = sum(h * w for h, w in case["refs"])
    lens = [n for n in (txt, img, cond) if n > 0]
    starts = [int(sum(lens[:i])) for i in range(len(lens))]
    mods = [(0.4 * ol.randn(seed + 30 + i, 3 * dim)).astype(np.float32) for i in range(len(lens))]
    inp.update(seg_start=np.array(starts, np.int32), seg_len=np.array(lens, np.int32), seg_mod=mods)
    return inp


def oracle_f3_block(inp, eps=1e-6, key_mask=None, nthreads=0):
    x = inp["x"].copy()
    o = ol.oracle()
    fn = o.orc_single_block_segments
    fn.restype = C.c_int
    fn.argtypes = [ol.f32p, ol.u16p, ol.u16p, ol.f32p, ol.f32p, ol.i32p, ol.i32p, C.c_void_p, C.c_int, ol.f32p, ol.f32p] + \
                  [C.c_int] * 4 + [C.c_float, ol.i32p_opt, C.c_int]
    n = len(inp["seg_mod"])
    mods = (C.c_void_p * n)(*[m.ctypes.data for m in inp["seg_mod"]])
    rc = fn(x, inp["w_in"], inp["w_out"], inp["norm_q"], inp["norm_k"], inp["seg_start"], inp["seg_len"], mods, n,
            inp["cos"], inp["sin"], inp["seq"], inp["dim"], inp["heads"], inp["mlp"], eps, key_mask, nthreads)
    assert rc == 0
    return x


# ---------------------------------------------------------------------------
# Z-Image block
# ---------------------------------------------------------------------------

ZI_SMALL = dict(name="zimage-block-small", family="zimage", heads=2, ff=704, txt=50, img=(9, 13), refs=[], eps=1e-5)
ZI_MID = dict(name="zimage-block-mid", family="zimage", heads=4, ff=1368, txt=40, img=(12, 11), refs=[], eps=1e-5)
ZI_30_HEADS = dict(name="zimage-block-30-heads", family="zimage", heads=30, ff=10240, txt=40, img=(8, 12), refs=[], eps=1e-5)

ZI_KEYS = ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k", "attn_norm1", "attn_norm2", "ffn_norm1", "ffn_norm2")


class ZImageWeights(C.Structure):
    """iris_b200_zimage_weights of include/iris_b200.h; orc_zimage_weights of
    oracle/iris_oracle.h has the same layout."""
    _fields_ = [(n, C.c_void_p) for n in ZI_KEYS]


def zi_positions(case):
    o = ol.oracle()
    seq = pc.seq_len(case)
    pos = np.zeros((seq, 3), np.int32)
    mask = np.zeros(seq, np.int32)
    assert o.orc_zi_positions(pos.reshape(-1), mask, case["img"][0], case["img"][1], case["txt"]) == seq
    return pos, mask


def zi_inputs(case, seed=91, modulated=True):
    H, ff = case["heads"], case["ff"]
    dim, seq = H * D, pc.seq_len(case)
    s = np.float32
    cos, sin, mask = pc.rope_tables(case)
    pos, full_mask = zi_positions(case)
    w = dict(
        qkv=ol.to_bf16(ol.randn(seed + 1, 3 * dim, dim) / s(np.sqrt(dim))),
        proj=ol.to_bf16(ol.randn(seed + 2, dim, dim) / s(np.sqrt(dim))),
        ff_in=ol.to_bf16(ol.randn(seed + 3, 2 * ff, dim) / s(np.sqrt(dim))),
        ff_out=ol.to_bf16(ol.randn(seed + 4, dim, ff) / s(np.sqrt(ff))),
        norm_q=(1.0 + 0.1 * ol.randn(seed + 5, D)).astype(s), norm_k=(1.0 + 0.1 * ol.randn(seed + 6, D)).astype(s))
    for i, k in enumerate(("attn_norm1", "attn_norm2", "ffn_norm1", "ffn_norm2")):
        w[k] = (1.0 + 0.1 * ol.randn(seed + 7 + i, dim)).astype(s)
    mod = (0.5 * ol.randn(seed + 20, 4 * dim)).astype(s) if modulated else None
    return dict(x=ol.randn(seed, seq, dim), w=w, mod=mod, cos=cos, sin=sin, mask=mask, pos=pos, full_mask=full_mask, seq=seq,
                dim=dim, heads=H, ff=ff)


def oracle_zi_block(inp, nthreads=0):
    x = inp["x"].copy()
    o = ol.oracle()
    fn = o.orc_zimage_block
    fn.restype = C.c_int
    fn.argtypes = [ol.f32p, C.POINTER(ZImageWeights), ol.f32p_opt, ol.f32p, ol.f32p] + [C.c_int] * 4 + [ol.i32p_opt, C.c_int]
    w = ZImageWeights(*[inp["w"][k].ctypes.data for k in ZI_KEYS])
    rc = fn(x, C.byref(w), inp["mod"], inp["cos"], inp["sin"], inp["seq"], inp["dim"], inp["heads"], inp["ff"], inp["mask"],
            nthreads)
    assert rc == 0
    return x
