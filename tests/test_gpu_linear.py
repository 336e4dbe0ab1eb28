"""The QKV projection with the prologue as its epilogue (tcgen05 GEMM) against
the CPU oracle: fp32 product of the bf16-rounded operands, rounded to bf16
(what the reference's cuBLAS GEMM stores), then the restated prologue
arithmetic of the reference's GPU kernel on the Q and K column blocks.

Bar: the GEMM's accumulation order differs from any reference's, so a product
that lies on a bf16 rounding boundary may round the other way: at least 98 %
of the elements must be bit-equal and no element may be off by more than two
bf16 steps of its head's largest value."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu

D = 128


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.check()


def oracle_linear(x, W, heads, cos, sin, eps):
    """bf16 bits of y; x [rows, in], W [out, in] bf16 bits."""
    xf, wf = ol.from_bf16(x).astype(np.float64), ol.from_bf16(W).astype(np.float64)
    y = ol.to_bf16((xf @ wf.T).astype(np.float32))
    if heads:
        o = ol.oracle()
        w1 = np.ones(D, np.float32)
        rows, out = y.shape
        y = np.ascontiguousarray(y)
        for blk in range(2):                       # Q heads, K heads
            o.orc_head_norm_rope_bf16(y.ctypes.data + blk * heads * D * 2, out, w1 * (1.0 + 0.25 * blk), cos, sin,
                                      rows, heads, D, eps, 0)
    return y


def run_linear(lib, rows, kin, out, heads, seed, ldy=None, eps=1e-6):
    ldy = ldy or out
    x = ol.to_bf16(ol.randn(seed, rows, kin))
    W = ol.to_bf16(ol.randn(seed + 1, out, kin) / np.sqrt(kin))
    ang = ol.randn(seed + 2, rows, 64) * 3.0
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    dx, dW = lib.to_device(x), lib.to_device(W)
    dcos, dsin = lib.to_device(cos), lib.to_device(sin)
    dwq, dwk = lib.to_device(np.ones(D, np.float32)), lib.to_device(np.full(D, 1.25, np.float32))
    dy = lib.to_device(np.full((rows, ldy), 0x7FC0, np.uint16))          # NaN canaries
    if heads:
        rc = lib.iris_b200_linear_qk_norm_rope(dy, ldy, dx, dW, rows, kin, out, heads, dwq, dwk, dcos, dsin, eps)
        assert rc == 0, rc
    else:
        assert ldy == out
        lib.iris_dev_linear_bf16(dy, dx, dW, rows, kin, out)
    got = lib.to_host(dy, (rows, ldy), np.uint16)
    lib.check()
    for p in (dx, dW, dcos, dsin, dwq, dwk, dy):
        lib.iris_dev_free(p)
    want = oracle_linear(x, W, heads, cos, sin, eps)
    assert (got[:, out:] == 0x7FC0).all()                                # nothing written past the row
    return got[:, :out], want


def check(got, want, heads=0):
    g, w = ol.from_bf16(got), ol.from_bf16(want)
    assert np.isfinite(g).all()
    equal = (got == want).mean()
    scale = np.maximum(np.abs(w).max(), 1.0)
    worst = np.abs(g - w).max()
    assert equal >= 0.98, equal
    assert worst <= 2 * 2.0 ** -8 * scale * 2, (worst, scale)


@pytest.mark.parametrize("rows,kin,out,heads", [
    (300, 256, 768, 2),          # Q | K | V of two heads, three N tiles, ragged rows
    (128, 64, 256, 1),           # one k-block, one tile
    (513, 1000, 1288, 3),        # K not a multiple of 64, N tail of 8 columns, 2.5 heads of plain columns
    (1000, 3072, 1536, 4),       # long reduction, many tiles per CTA
])
def test_projection_with_prologue_epilogue(lib, rows, kin, out, heads):
    got, want = run_linear(lib, rows, kin, out, heads, seed=rows + out)
    check(got, want, heads)


def test_plain_linear_is_the_reference_entry_point(lib):
    got, want = run_linear(lib, 257, 512, 640, 0, seed=7)
    check(got, want)


def test_output_row_stride(lib):
    got, want = run_linear(lib, 200, 256, 512, 1, seed=9, ldy=520)
    check(got, want, 1)


def test_klein4b_projection_at_full_size_on_sampled_rows(lib):
    """4608 x 3072 -> 9216 (the double block's QKV GEMM): sampled rows
    against the oracle, all columns."""
    rows, kin, heads = 4608, 3072, 24
    out = 3 * heads * D
    x = ol.to_bf16(ol.randn(21, rows, kin))
    W = ol.to_bf16(ol.randn(22, out, kin) / np.sqrt(kin))
    ang = ol.randn(23, rows, 64)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    dx, dW, dcos, dsin = lib.to_device(x), lib.to_device(W), lib.to_device(cos), lib.to_device(sin)
    dwq, dwk = lib.to_device(np.ones(D, np.float32)), lib.to_device(np.full(D, 1.25, np.float32))
    dy = lib.alloc(rows * out * 2)
    assert lib.iris_b200_linear_qk_norm_rope(dy, out, dx, dW, rows, kin, out, heads, dwq, dwk, dcos, dsin, 1e-6) == 0
    got = lib.to_host(dy, (rows, out), np.uint16)
    lib.check()
    for p in (dx, dW, dcos, dsin, dwq, dwk, dy):
        lib.iris_dev_free(p)
    sel = np.unique(np.concatenate([[0, 127, 128, 4607], np.random.default_rng(3).integers(0, rows, 60)]))
    want = oracle_linear(np.ascontiguousarray(x[sel]), W, heads, np.ascontiguousarray(cos[sel]),
                         np.ascontiguousarray(sin[sel]), 1e-6)
    check(got[sel], want, heads)


def test_argument_checks(lib):
    assert lib.iris_b200_linear_qk_norm_rope(16, 256, 16, 16, 4, 64, 256, 2, 16, 16, 16, 16, 1e-6) == 1   # 2 heads need 512 columns
    lib.iris_b200_clear_error()
    assert lib.iris_b200_linear_qk_norm_rope(16, 256, 16, 16, 4, 60, 256, 1, 16, 16, 16, 16, 1e-6) == 6   # in % 8
    lib.iris_b200_clear_error()
    assert lib.iris_b200_linear_qk_norm_rope(16, 250, 16, 16, 4, 64, 256, 1, 16, 16, 16, 16, 1e-6) == 1   # ldy < out
    lib.iris_b200_clear_error()
