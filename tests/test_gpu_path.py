"""Parity of the CUDA path against the CPU oracle, through the C-ABI.

Gate (per head): max |gpu - cpu| <= 2e-2 and cosine >= 0.9999 for bf16 inputs
with fp32 accumulation; the prologue alone is held to bf16 resolution."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol
import path_cases as pc

pytestmark = pytest.mark.gpu

D = 128
MAX_ABS, MIN_COS = 2e-2, 0.9999
TC, GEN = 1, 2


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.check()


def gate(res):
    assert res["max_abs"] <= MAX_ABS and res["min_cos"] >= MIN_COS, (
        res["max_abs"], res["min_cos"], res["per_head_max"], res["per_head_cos"])
    # |x| <= sqrt(128) after the norm, bf16 has 8 bits of mantissa
    assert res["prologue_max_abs"] <= 11.4 * 2.0 ** -8


# ---------------------------------------------------------------------------
# runtime
# ---------------------------------------------------------------------------

def test_runtime_alloc_copy_cast(lib):
    assert lib.iris_dev_available() == 1 and lib.iris_dev_init() == 1
    assert b"B200" in lib.iris_dev_name() or lib.iris_dev_name() != b"none"
    p0 = lib.iris_dev_alloc(0)
    assert p0
    lib.iris_dev_free(p0)
    lib.iris_dev_free(None)
    x = ol.randn(3, 1000, 37)
    d = lib.to_device(x)
    assert np.array_equal(lib.to_host(d, x.shape, np.float32), x)
    b = lib.alloc(x.size * 2)
    lib.iris_dev_f32_to_bf16(b, d, x.size)
    assert np.array_equal(lib.to_host(b, x.shape, np.uint16), ol.to_bf16(x))
    # strided upload: 5 rows of 12 bytes from stride 20 to stride 16
    src = np.arange(100, dtype=np.uint8)
    dst = lib.alloc(80)
    lib.iris_dev_upload(dst, np.zeros(80, np.uint8).ctypes.data, 80)
    lib.iris_dev_upload_2d(dst, 16, src.ctypes.data, 20, 12, 5)
    got = lib.to_host(dst, (5, 16), np.uint8)
    for r in range(5):
        assert np.array_equal(got[r, :12], src[20 * r:20 * r + 12]) and not got[r, 12:].any()
    for p in (d, b, dst):
        lib.iris_dev_free(p)
    lib.check()


# ---------------------------------------------------------------------------
# prologue
# ---------------------------------------------------------------------------

def prologue_case(lib, seq, heads, hd, ld, split_half, fused, eps=1e-6, col0=0):
    o = ol.oracle()
    x = ol.randn(100 + seq + heads, seq, ld) * np.float32(1.7)
    xb = ol.to_bf16(x)
    w = (1.0 + 0.25 * ol.randn(7, hd)).astype(np.float32)
    w2 = (1.0 + 0.25 * ol.randn(8, hd)).astype(np.float32)
    ang = ol.randn(9, seq, hd // 2) * np.float32(3.0)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    dx, dw, dw2, dc, ds = (lib.to_device(a) for a in (xb, w, w2, cos, sin))
    width = heads * hd
    pq = C.c_void_p(dx + col0 * 2)
    pk = C.c_void_p(dx + (col0 + width) * 2)
    want = xb.copy()
    wq = want[:, col0:]
    o.orc_head_norm_rope_bf16(wq.ctypes.data, ld, w, cos, sin, seq, heads, hd, eps, split_half)
    if fused:
        assert lib.iris_b200_qk_norm_rope(pq, pk, ld, dw, dw2, dc, ds, seq, heads, hd, eps, split_half) == 0
        wk = want[:, col0 + width:]
        o.orc_head_norm_rope_bf16(wk.ctypes.data, ld, w2, cos, sin, seq, heads, hd, eps, split_half)
    else:
        lib.iris_dev_head_norm_rope(pq, ld, dw, dc, ds, seq, heads, hd, eps, split_half)
    got = lib.to_host(dx, xb.shape, np.uint16)
    lib.check()
    for p in (dx, dw, dw2, dc, ds):
        lib.iris_dev_free(p)
    # untouched columns stay bit-identical; touched ones within one bf16 ulp
    g, wv = ol.from_bf16(got), ol.from_bf16(want)
    touched = np.zeros(ld, bool)
    touched[col0:col0 + width * (2 if fused else 1)] = True
    assert np.array_equal(got[:, ~touched], xb[:, ~touched])
    err = np.abs(g - wv)
    tol = np.maximum(np.abs(wv), 2.0 ** -6) * 2.0 ** -7
    assert (err <= tol).all(), float((err / tol).max())
    assert (got != want).mean() < 0.02          # rsqrt vs 1/sqrt: rare last-bit flips only


@pytest.mark.parametrize("split_half", [0, 1])
@pytest.mark.parametrize("fused", [True, False])
def test_prologue_fast_kernel(lib, split_half, fused):
    prologue_case(lib, 517, 6, 128, 3 * 6 * 128 + 64, split_half, fused, col0=8)


def test_prologue_tiny_and_empty(lib):
    prologue_case(lib, 1, 1, 128, 256, 0, True)
    prologue_case(lib, 3, 5, 128, 2 * 5 * 128, 0, True)
    lib.iris_dev_head_norm_rope(None, 128, None, None, None, 0, 4, 128, 1e-6, 0)   # seq 0: no-op
    assert lib.iris_b200_last_error() == 0


@pytest.mark.parametrize("hd,ld,col0", [(64, 2 * 4 * 64, 0), (128, 4 * 128 + 6, 3), (512, 512, 0)])
def test_prologue_general_kernel(lib, hd, ld, col0):
    heads = 1 if hd == 512 else 4
    prologue_case(lib, 37, heads, hd, max(ld, col0 + heads * hd), 1 if hd == 64 else 0, False, col0=col0)


# ---------------------------------------------------------------------------
# attention: small cases of every family, both kernels
# ---------------------------------------------------------------------------

SMALL = [pc.FLUX_SMALL, pc.FLUX_REF_SMALL, pc.FLUX3_SMALL, pc.ZIMAGE_SMALL]


@pytest.mark.parametrize("case", SMALL, ids=lambda c: c["name"])
@pytest.mark.parametrize("kernel", [GEN, TC], ids=["generic", "tcgen05"])
def test_small_cases(lib, case, kernel):
    gate(pc.run_case(lib, case, kernel=kernel))


def test_unfused_prologue_gives_the_same_bits(lib):
    a = pc.run_case(lib, pc.FLUX_SMALL, kernel=TC, fused_prologue=True)
    b = pc.run_case(lib, pc.FLUX_SMALL, kernel=TC, fused_prologue=False)
    assert np.array_equal(a["out"], b["out"])


def attention_raw(lib, seq_q, seq_k, heads, kernel, kv_heads=None, hd=128, causal=0, mask=None,
                  pad=0, seed=0, scale=None):
    """Attention on plain (already normalised) bf16 tensors, out vs oracle."""
    kv_heads = kv_heads or heads
    ldi = max(heads, kv_heads) * hd + pad
    q = np.zeros((seq_q, ldi), np.float32)
    k = np.zeros((seq_k, ldi), np.float32)
    v = np.zeros((seq_k, ldi), np.float32)
    q[:, :heads * hd] = ol.randn(seed + 1, seq_q, heads * hd)
    k[:, :kv_heads * hd] = ol.randn(seed + 2, seq_k, kv_heads * hd)
    v[:, :kv_heads * hd] = ol.randn(seed + 3, seq_k, kv_heads * hd)
    qb, kb, vb = ol.to_bf16(q), ol.to_bf16(k), ol.to_bf16(v)
    ldo = heads * hd + pad
    dq, dk, dv = lib.to_device(qb), lib.to_device(kb), lib.to_device(vb)
    dout = lib.to_device(np.full((max(seq_q, 1), ldo), 0x7FC0, np.uint16))      # NaN canary
    dm = lib.to_device(np.ascontiguousarray(mask, np.int32)) if mask is not None else None
    scale = scale if scale is not None else 1.0 / np.sqrt(hd)
    rc = lib.iris_b200_attention_ex(dout, ldo, dq, dk, dv, ldi, seq_q, seq_k, heads, kv_heads, hd,
                                    scale, causal, dm, kernel)
    assert rc == 0, rc
    raw = lib.to_host(dout, (max(seq_q, 1), ldo), np.uint16)
    lib.check()
    for p in (dq, dk, dv, dout, dm):
        if p:
            lib.iris_dev_free(p)
    got = ol.from_bf16(raw)[:seq_q, :heads * hd]
    if pad:
        assert (raw[:, heads * hd:] == 0x7FC0).all()       # nothing written outside the slice
    want = ol.dev_attention(ol.from_bf16(qb)[:, :heads * hd], ol.from_bf16(kb)[:, :kv_heads * hd],
                            ol.from_bf16(vb)[:, :kv_heads * hd], heads, kv_heads, hd, scale, causal, mask)
    return got, want


def check_raw(got, want, heads, hd=128):
    assert np.isfinite(got).all()
    if got.size == 0:
        return
    mx, cs = ol.compare_heads(got, want, heads, hd)
    live = np.abs(want).reshape(want.shape[0], heads, hd).sum((0, 2)) > 0
    assert mx.max() <= MAX_ABS, mx
    assert (cs[live] >= MIN_COS).all(), cs


@pytest.mark.parametrize("seq", [1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, 383, 640])
@pytest.mark.parametrize("kernel", [GEN, TC], ids=["generic", "tcgen05"])
def test_ragged_lengths(lib, seq, kernel):
    got, want = attention_raw(lib, seq, seq, 2, kernel, seed=seq)
    check_raw(got, want, 2)


@pytest.mark.parametrize("seq_q,seq_k", [(1, 300), (300, 1), (130, 700), (513, 129)])
@pytest.mark.parametrize("kernel", [GEN, TC], ids=["generic", "tcgen05"])
def test_rectangular(lib, seq_q, seq_k, kernel):
    got, want = attention_raw(lib, seq_q, seq_k, 3, kernel, seed=seq_q + seq_k, pad=8)
    check_raw(got, want, 3)


@pytest.mark.parametrize("kernel", [GEN, TC], ids=["generic", "tcgen05"])
def test_key_mask_and_fully_masked_rows(lib, kernel):
    rng = np.random.default_rng(3)
    mask = (rng.random(419) > 0.3).astype(np.int32)
    mask[128:256] = 0                      # a whole key tile hidden
    mask[0] = 0
    got, want = attention_raw(lib, 300, 419, 2, kernel, mask=mask, seed=11)
    check_raw(got, want, 2)
    # last 17 keys masked
    m2 = np.ones(419, np.int32); m2[-17:] = 0
    got, want = attention_raw(lib, 300, 419, 2, kernel, mask=m2, seed=12)
    check_raw(got, want, 2)
    # no valid key at all: zeros, not NaN
    got, want = attention_raw(lib, 140, 200, 2, kernel, mask=np.zeros(200, np.int32), seed=13)
    assert not got.any() and not want.any()
    # first tile hidden, later tile visible: exercises the -inf reference
    m3 = np.ones(400, np.int32); m3[:130] = 0
    got, want = attention_raw(lib, 200, 400, 2, kernel, mask=m3, seed=14)
    check_raw(got, want, 2)


@pytest.mark.parametrize("seq_q,seq_k,heads", [(700, 1500, 5), (257, 513, 2), (130, 4100, 3)])
def test_key_split_launches(lib, seq_q, seq_k, heads):
    """Few query blocks and four or more key tiles: the tcgen05 kernel gives
    each half of the keys to a CTA of its own and the later one merges."""
    got, want = attention_raw(lib, seq_q, seq_k, heads, TC, seed=seq_q + 7 * seq_k)
    check_raw(got, want, heads)
    # one half of the keys masked out entirely, then a ragged mix
    for lo, hi in ((0, seq_k // 2 + 64), (seq_k // 2 - 30, seq_k)):
        m = np.ones(seq_k, np.int32)
        m[lo:hi] = 0
        m[5::7] = 0
        got, want = attention_raw(lib, seq_q, seq_k, heads, TC, mask=m, seed=seq_q + lo)
        check_raw(got, want, heads)


def test_use_stream_runs_calls_side_by_side(lib):
    """Two independent attention calls on two caller-owned streams, switched
    without synchronisation, both correct once the streams are drained."""
    rt = C.CDLL("libcudart.so.12")
    streams = [C.c_void_p(), C.c_void_p()]
    for st in streams:
        assert rt.cudaStreamCreateWithFlags(C.byref(st), 1) == 0           # non-blocking
    heads = 2
    jobs = []
    for i, (sq, sk) in enumerate(((600, 900), (300, 2000))):
        q, k, v = (ol.to_bf16(ol.randn(50 + 3 * i + j, n, heads * D)) for j, n in enumerate((sq, sk, sk)))
        dq, dk, dv = lib.to_device(q), lib.to_device(k), lib.to_device(v)
        dout = lib.alloc(sq * heads * D * 2)
        jobs.append((q, k, v, dq, dk, dv, dout, sq, sk))
    lib.iris_dev_sync()
    for rep in range(3):
        for st, (q, k, v, dq, dk, dv, dout, sq, sk) in zip(streams, jobs):
            assert lib.iris_b200_use_stream(st) == 0
            lib.iris_dev_attention(dout, heads * D, dq, dk, dv, heads * D, sq, sk, heads, heads, D,
                                   1.0 / np.sqrt(D), 0, None)
    assert lib.iris_b200_use_stream(None) == 0
    for st in streams:
        assert rt.cudaStreamSynchronize(st) == 0
    for q, k, v, dq, dk, dv, dout, sq, sk in jobs:
        got = ol.from_bf16(lib.to_host(dout, (sq, heads * D), np.uint16))
        want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), heads)
        check_raw(got, want, heads)
        for p in (dq, dk, dv, dout):
            lib.iris_dev_free(p)
    for st in streams:
        rt.cudaStreamDestroy(st)
    lib.check()


def test_masked_calls_on_two_streams_keep_their_own_masks(lib):
    """Key masks are packed into per-stream scratch: two masked calls that
    overlap on two streams must not see each other's bits; ten streams in a
    row exercise the recycling of the scratch sets."""
    heads = 2
    streams = [lib.iris_b200_stream_create() for _ in range(2)]
    jobs = []
    for i, (sq, sk) in enumerate(((500, 1500), (400, 1400))):
        q, k, v = (ol.to_bf16(ol.randn(80 + 3 * i + j, n, heads * D)) for j, n in enumerate((sq, sk, sk)))
        mask = (ol.randn(90 + i, 1, sk)[0] > (0.0 if i else -0.8)).astype(np.int32)      # different patterns
        mask[:3] = 1
        jobs.append((q, k, v, mask, lib.to_device(q), lib.to_device(k), lib.to_device(v), lib.to_device(mask),
                     lib.alloc(sq * heads * D * 2), sq, sk))
    lib.iris_dev_sync()
    for rep in range(4):
        for st, (q, k, v, mask, dq, dk, dv, dm, dout, sq, sk) in zip(streams, jobs):
            assert lib.iris_b200_use_stream(st) == 0
            lib.iris_dev_attention(dout, heads * D, dq, dk, dv, heads * D, sq, sk, heads, heads, D,
                                   1.0 / np.sqrt(D), 0, dm)
    assert lib.iris_b200_use_stream(None) == 0
    for st in streams:
        assert lib.iris_b200_stream_sync(st) == 0
    for q, k, v, mask, dq, dk, dv, dm, dout, sq, sk in jobs:
        got = ol.from_bf16(lib.to_host(dout, (sq, heads * D), np.uint16))
        want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), heads, key_mask=mask)
        check_raw(got, want, heads)
    # more streams than the library keeps scratch sets for
    q, k, v, mask, dq, dk, dv, dm, dout, sq, sk = jobs[0]
    want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), heads, key_mask=mask)
    for i in range(10):
        st = lib.iris_b200_stream_create()
        assert lib.iris_b200_use_stream(st) == 0
        lib.iris_dev_attention(dout, heads * D, dq, dk, dv, heads * D, sq, sk, heads, heads, D, 1.0 / np.sqrt(D), 0, dm)
        assert lib.iris_b200_stream_sync(st) == 0
        assert lib.iris_b200_use_stream(None) == 0
        check_raw(ol.from_bf16(lib.to_host(dout, (sq, heads * D), np.uint16)), want, heads)
        lib.iris_b200_stream_destroy(st)
    for job in jobs:
        for p in job[4:9]:
            lib.iris_dev_free(p)
    for st in streams:
        lib.iris_b200_stream_destroy(st)
    lib.check()


def test_empty_sequences(lib):
    got, _ = attention_raw(lib, 0, 50, 2, 0)
    assert got.size == 0
    got, want = attention_raw(lib, 33, 0, 2, 0)
    assert not got.any()


def test_large_logits_force_rescale(lib):
    """Growing row maxima across key tiles: the lazy rescale must trigger."""
    seq_q, seq_k, H = 256, 1024, 1
    q = ol.randn(1, seq_q, D)
    k = ol.randn(2, seq_k, D)
    k *= np.linspace(0.2, 6.0, seq_k, dtype=np.float32)[:, None]     # later keys score higher
    v = ol.randn(3, seq_k, D)
    qb, kb, vb = ol.to_bf16(q), ol.to_bf16(k), ol.to_bf16(v)
    dq, dk, dv = lib.to_device(qb), lib.to_device(kb), lib.to_device(vb)
    dout = lib.alloc(seq_q * D * 2)
    outs = []
    for kernel in (GEN, TC):
        assert lib.iris_b200_attention_ex(dout, D, dq, dk, dv, D, seq_q, seq_k, H, H, D,
                                          1.0 / np.sqrt(D), 0, None, kernel) == 0
        outs.append(ol.from_bf16(lib.to_host(dout, (seq_q, D), np.uint16)))
    lib.check()
    for p in (dq, dk, dv, dout):
        lib.iris_dev_free(p)
    want = ol.dev_attention(ol.from_bf16(qb), ol.from_bf16(kb), ol.from_bf16(vb), H)
    for got in outs:
        check_raw(got, want, H)


# ---------------------------------------------------------------------------
# the other argument domains of the same op (general kernel)
# ---------------------------------------------------------------------------

def test_gqa_causal_masked(lib):
    """Text-encoder style: 8 query heads on 2 kv heads, causal, padding mask."""
    mask = np.ones(90, np.int32); mask[70:] = 0
    got, want = attention_raw(lib, 90, 90, 8, 0, kv_heads=2, causal=1, mask=mask, seed=21)
    check_raw(got, want, 8)
    assert lib.iris_b200_attention_kernel_for(16, 1024, 16, 16, 16, 1024, 8, 2, 128, 1) == GEN


@pytest.mark.parametrize("hd,heads", [(64, 4), (512, 1), (96, 2), (72, 3), (65, 2)])
def test_other_head_dims(lib, hd, heads):
    got, want = attention_raw(lib, 77, 130, heads, 0, hd=hd, seed=hd)
    check_raw(got, want, heads, hd)


def test_unaligned_views_take_the_general_kernel(lib):
    got, want = attention_raw(lib, 70, 70, 2, 0, pad=2, seed=5)      # ldi % 8 != 0
    check_raw(got, want, 2)
    rc = lib.iris_b200_attention_ex(16, 258, 16, 16, 16, 258, 1, 1, 2, 2, 128, 0.1, 0, None, TC)
    assert rc == 6                                                    # EUNSUPPORTED
    lib.iris_b200_clear_error()
    assert lib.iris_b200_attention_ex(None, 256, 16, 16, 16, 256, 1, 1, 2, 2, 128, 0.1, 0, None, 0) == 1
    lib.iris_b200_clear_error()


# ---------------------------------------------------------------------------
# host-pointer fp32 surface
# ---------------------------------------------------------------------------

def test_host_flash_attention(lib):
    H = 4
    q, k, v = ol.randn(1, 300, H * D), ol.randn(2, 450, H * D), ol.randn(3, 450, H * D)
    out = np.zeros_like(q)
    lib.iris_flash_attention(out.ctypes.data, q.ctypes.data, k.ctypes.data, v.ctypes.data,
                             300, 450, H, D, 1 / np.sqrt(D))
    lib.check()
    want = np.zeros_like(q)
    ol.oracle().orc_flash_attention(want, q, k, v, 300, 450, H, D, 1 / np.sqrt(D))
    mx, cs = ol.compare_heads(out, want, H)
    assert mx.max() <= MAX_ABS and cs.min() >= MIN_COS


def test_host_batched_attention(lib):
    B, H, Sq, Sk = 2, 3, 70, 200
    q, k, v = ol.randn(4, B, H, Sq, D), ol.randn(5, B, H, Sk, D), ol.randn(6, B, H, Sk, D)
    out = np.zeros_like(q)
    lib.iris_attention(out.ctypes.data, q.ctypes.data, k.ctypes.data, v.ctypes.data, B, H, Sq, Sk, D, 1 / np.sqrt(D))
    lib.check()
    want = np.zeros_like(q)
    ol.oracle().orc_attention(want.reshape(-1), q.reshape(-1), k.reshape(-1), v.reshape(-1), B, H, Sq, Sk, D, 1 / np.sqrt(D))
    assert np.abs(out - want).max() <= MAX_ABS
    a, b = out.reshape(B * H, -1), want.reshape(B * H, -1)
    cos = (a * b).sum(1) / np.sqrt((a * a).sum(1) * (b * b).sum(1))
    assert cos.min() >= MIN_COS


def test_host_softmax_and_rope(lib):
    o = ol.oracle()
    x = ol.randn(1, 50, 777) * np.float32(4.0)
    want = x.copy()
    o.orc_softmax(want.reshape(-1), 50, 777)
    lib.iris_softmax(x.ctypes.data, 50, 777)
    np.testing.assert_allclose(x, want, rtol=0, atol=2e-6)
    pos = np.arange(0, 200, 7, dtype=np.int32)
    fr = np.zeros((pos.size, 32, 2), np.float32)
    wf = np.zeros_like(fr)
    lib.iris_compute_rope_freqs(fr.ctypes.data, pos.ctypes.data, pos.size, 64, 10000.0)
    o.orc_compute_rope_freqs(wf.reshape(-1), pos, pos.size, 64, 10000.0)
    np.testing.assert_allclose(fr, wf, rtol=0, atol=2e-5)
    y = ol.randn(2, 2, pos.size, 3, 64)
    wy = y.copy()
    lib.iris_apply_rope(y.ctypes.data, wf.ctypes.data, 2, pos.size, 3, 64)
    o.orc_apply_rope(wy.reshape(-1), wf.reshape(-1), 2, pos.size, 3, 64)
    np.testing.assert_allclose(y, wy, rtol=0, atol=2e-6)
    lib.check()


def test_c_host_program_matches_the_oracle(lib, tmp_path):
    """The plain-C program written against include/iris_dev.h (prologue on Q
    and K, attention on the fused-QKV slices, as the reference's block code
    calls them) gives the oracle's result within the gate."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "iris.c_b200")
    exe = os.path.join(pkg, "build", "block_attention")
    if not os.path.exists(exe):          # normally built by build() / the CPU suite beforehand
        subprocess.check_call(["make", "-C", pkg, "example"], stdout=subprocess.DEVNULL)
    case = pc.FLUX_REF_SMALL
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    pc.write_block_input(inp, case)
    r = subprocess.run([exe, str(inp), str(out)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    H = case["heads"]
    got = ol.from_bf16(np.fromfile(out, np.uint16).reshape(pc.seq_len(case), H * D))
    want, _, _, rows = pc.oracle_case(case)
    mx, cs = ol.compare_heads(got, want, H, D, rows)
    assert mx.max() <= MAX_ABS and cs.min() >= MIN_COS, (mx, cs)
