"""GPU tests of the operators around the attention path and of one FLUX.2
single-stream block, through the C-ABI, against the CPU restatement (which the
CPU tests pin to the reference's single_block_forward) and, where it is built,
against the reference's own CUDA backend issuing its eight-call sequence on the
same device buffers."""
import ctypes as C

import numpy as np
import pytest

import block_cases as bc
import oracle_lib as ol

pytestmark = pytest.mark.gpu

REL_MAX, MIN_COS = 2e-2, 0.9999


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.check()


def bf16_ulp(x):
    return np.maximum(np.abs(x), 2.0 ** -126) * 2.0 ** -7


class Dev:
    """Device copies that are freed together."""

    def __init__(self, lib):
        self.lib, self.ptrs = lib, []

    def put(self, arr):
        p = self.lib.to_device(arr)
        self.ptrs.append(p)
        return p

    def new(self, nbytes):
        p = self.lib.alloc(nbytes)
        self.ptrs.append(p)
        return p

    def free(self):
        for p in self.ptrs:
            self.lib.iris_dev_free(p)
        self.ptrs = []


@pytest.mark.parametrize("rows,dim", [(37, 3072), (300, 512), (5, 4100), (6, 1030), (3, 4096)])
def test_layer_norm_mod(lib, rows, dim):
    o = ol.oracle()
    x = (ol.randn(rows + dim, rows, dim) * 2 + 0.5).astype(np.float32)
    shift, scale = ol.randn(1, dim), (ol.randn(2, dim) * np.float32(0.3)).astype(np.float32)
    d = Dev(lib)
    try:
        dx, dsh, dsc, dout = d.put(x), d.put(shift), d.put(scale), d.new(rows * dim * 2)
        for sh, sc, psh, psc in ((shift, scale, dsh, dsc), (None, scale, None, dsc), (shift, None, dsh, None)):
            lib.iris_dev_layer_norm_mod(dout, dx, psh, psc, rows, dim, 1e-6)
            got = lib.to_host(dout, (rows, dim), np.uint16)
            lib.check()
            want = np.zeros((rows, dim), np.uint16)
            o.orc_layer_norm_mod(want, x, sh, sc, rows, dim, 1e-6)
            fw = ol.from_bf16(want)
            assert (got != want).mean() < 0.02
            assert (np.abs(ol.from_bf16(got) - fw) <= bf16_ulp(fw) * 1.01).all()
    finally:
        d.free()


@pytest.mark.parametrize("rows,cols,ldi,ldo,off", [(33, 1024, 2304, 1280, 1152), (9, 40, 100, 56, 50)])
def test_swiglu(lib, rows, cols, ldi, ldo, off):
    o = ol.oracle()
    src = ol.to_bf16(ol.randn(rows, rows, ldi) * 4)
    src[0, :8] = ol.to_bf16(np.array([-100, -60, -20, 0, 20, 60, 100, 1e-3], np.float32))
    d = Dev(lib)
    try:
        dsrc, dout = d.put(src), d.put(np.zeros((rows, ldo), np.uint16))
        lib.iris_dev_swiglu(dout, ldo, dsrc, dsrc + 2 * off, ldi, rows, cols)
        got = lib.to_host(dout, (rows, ldo), np.uint16)
        lib.check()
    finally:
        d.free()
    want = np.zeros((rows, ldo), np.uint16)
    o.orc_swiglu(want.ctypes.data, ldo, src.ctypes.data, src.ctypes.data + 2 * off, ldi, rows, cols)
    fw = ol.from_bf16(want)
    assert (got != want).mean() < 0.01
    assert (np.abs(ol.from_bf16(got) - fw) <= bf16_ulp(fw) * 1.01).all()
    assert not got[:, cols:].any()


@pytest.mark.parametrize("rows,dim", [(65, 3072), (7, 50)])
def test_residual(lib, rows, dim):
    x, a, gate = ol.randn(1, rows, dim), ol.randn(2, rows, dim), ol.randn(3, dim)
    d = Dev(lib)
    try:
        da, dg = d.put(a), d.put(gate)
        for g, pg in ((gate, dg), (None, None)):
            dx = d.put(x)
            lib.iris_dev_residual(dx, da, pg, rows, dim)
            got = lib.to_host(dx, (rows, dim), np.float32)
            lib.check()
            want = x.astype(np.float64) + (g if g is not None else 1.0) * a.astype(np.float64)
            np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    finally:
        d.free()


@pytest.mark.parametrize("rows,cin,cout", [(200, 512, 264), (129, 1280, 512), (1, 64, 8)])
def test_linear_f32_and_linear_residual(lib, rows, cin, cout):
    o = ol.oracle()
    a = ol.to_bf16(ol.randn(rows, rows, cin))
    W = ol.to_bf16(ol.randn(cin, cout, cin) / np.float32(np.sqrt(cin)))
    x0, gate = ol.randn(5, rows, cout), ol.randn(6, cout)
    want = np.zeros((rows, cout), np.float32)
    o.orc_linear(want, cout, a, cin, W, cin, rows, cin, cout, 0)
    d = Dev(lib)
    try:
        da, dW, dg, dy = d.put(a), d.put(W), d.put(gate), d.new(rows * cout * 4)
        lib.iris_dev_linear_f32(dy, da, dW, rows, cin, cout)
        got = lib.to_host(dy, (rows, cout), np.float32)
        lib.check()
        np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-4)
        for g, pg in ((gate, dg), (None, None)):
            dx = d.put(x0)
            assert lib.iris_b200_linear_residual(dx, cout, da, cin, dW, cin, pg, rows, cin, cout) == 0
            got = lib.to_host(dx, (rows, cout), np.float32)
            lib.check()
            np.testing.assert_allclose(got, x0 + (g if g is not None else 1.0) * want, rtol=2e-4, atol=4e-4)
    finally:
        d.free()


def test_linear_residual_argument_checks(lib):
    d = Dev(lib)
    try:
        p = d.new(1 << 16)
        assert lib.iris_b200_linear_residual(None, 64, p, 64, p, 64, None, 8, 64, 64) == 1
        assert lib.iris_b200_linear_residual(p, 32, p, 64, p, 64, None, 8, 64, 64) == 1      # ldx < out
        assert lib.iris_b200_linear_residual(p, 64, p, 60, p, 64, None, 8, 64, 64) == 1      # lda < in
        assert lib.iris_b200_linear_residual(p, 64, p, 68, p, 64, None, 8, 64, 64) != 0      # lda % 8
        assert lib.iris_b200_single_block(p, p, p, p, p, p, p, p, p, 8, 200, 2, 64, None) == 1   # dim != heads * 128
        assert lib.iris_b200_single_block(p, p + 16, p, p, p, p, p, p, p, 8, 256, 2, 64, None) == 1   # scratch alignment
        assert lib.iris_b200_single_block_scratch_bytes(8, 0, 64) == 0
        lib.iris_b200_clear_error()
    finally:
        d.free()


def device_block(lib, inp, key_mask=None, calls=1):
    d = Dev(lib)
    try:
        dx = d.put(inp["x"])
        nbytes = lib.iris_b200_single_block_scratch_bytes(inp["seq"], inp["dim"], inp["mlp"])
        assert nbytes > 0
        scratch = d.new(nbytes)
        args = [d.put(inp[k]) for k in ("w_in", "w_out", "norm_q", "norm_k", "mod", "cos", "sin")]
        dm = d.put(np.ascontiguousarray(key_mask, np.int32)) if key_mask is not None else None
        for _ in range(calls):
            rc = lib.iris_b200_single_block(dx, scratch, *args, inp["seq"], inp["dim"], inp["heads"], inp["mlp"], dm)
            assert rc == 0
        out = lib.to_host(dx, inp["x"].shape, np.float32)
        lib.check()
        return out
    finally:
        d.free()


@pytest.mark.parametrize("case", [bc.SMALL, bc.MID, bc.ODD_HEADS, bc.KLEIN4B_SHORT], ids=lambda c: c["name"])
def test_single_block_against_the_restatement(lib, case):
    inp = bc.block_inputs(case)
    got = device_block(lib, inp)
    rel, cos = bc.delta_metrics(got, bc.oracle_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_single_block_against_the_recorded_reference(lib):
    """Straight against the committed output of the reference's CPU block."""
    import os
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.block_inputs(bc.SMALL)
    rel, cos = bc.delta_metrics(device_block(lib, inp), gold[bc.SMALL["name"]], inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_single_block_with_key_mask(lib):
    inp = bc.block_inputs(bc.MID)
    mask = np.ones(inp["seq"], np.int32)
    mask[10:40] = 0
    got = device_block(lib, inp, mask)
    rel, cos = bc.delta_metrics(got, bc.oracle_block(inp, mask), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)
    assert not np.array_equal(got, device_block(lib, inp))


def test_two_blocks_in_a_row_reuse_the_scratch(lib):
    """The hidden state is updated in place: a second call continues from the first."""
    inp = bc.block_inputs(bc.SMALL)
    twice = device_block(lib, inp, calls=2)
    x1 = bc.oracle_block(inp)
    x2 = bc.oracle_block(dict(inp, x=x1))
    rel, cos = bc.delta_metrics(twice, x2, inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_single_block_against_the_reference_cuda_sequence(lib):
    """The reference's device forward issues eight calls per single block
    (iris_transformer_flux.c:3828-3845); its own CUDA backend runs them here on
    the same inputs. Same arithmetic rules, so the results must sit far inside
    the gate."""
    ref = ol.ref_cuda()
    if ref is None:
        pytest.skip("oracle/_ref/libiris_ref_cuda.so not built")
    assert ref.iris_dev_init() == 1
    case = bc.KLEIN4B_SHORT
    inp = bc.block_inputs(case)
    seq, dim, H, mlp = inp["seq"], inp["dim"], inp["heads"], inp["mlp"]
    ldh, ldc = 3 * dim + 2 * mlp, dim + mlp
    ours = device_block(lib, inp)
    d = Dev(lib)
    try:
        x, mod = d.put(inp["x"]), d.put(inp["mod"])
        w_in, w_out, nq, nk = d.put(inp["w_in"]), d.put(inp["w_out"]), d.put(inp["norm_q"]), d.put(inp["norm_k"])
        cos, sin = d.put(inp["cos"]), d.put(inp["sin"])
        norm, h, cat, out = d.new(seq * dim * 2), d.new(seq * ldh * 2), d.new(seq * ldc * 2), d.new(seq * dim * 4)
        lib.iris_dev_sync()
        ref.iris_dev_layer_norm_mod(norm, x, mod, mod + 4 * dim, seq, dim, 1e-6)
        ref.iris_dev_linear_bf16(h, norm, w_in, seq, dim, ldh)
        ref.iris_dev_head_norm_rope(h, ldh, nq, cos, sin, seq, H, 128, 1e-6, 0)
        ref.iris_dev_head_norm_rope(h + 2 * dim, ldh, nk, cos, sin, seq, H, 128, 1e-6, 0)
        ref.iris_dev_attention(cat, ldc, h, h + 2 * dim, h + 4 * dim, ldh, seq, seq, H, H, 128, 1.0 / np.sqrt(128.0), 0, None)
        ref.iris_dev_swiglu(cat + 2 * dim, ldc, h + 2 * 3 * dim, h + 2 * (3 * dim + mlp), ldh, seq, mlp)
        ref.iris_dev_linear_f32(out, cat, w_out, seq, ldc, dim)
        ref.iris_dev_residual(x, out, mod + 8 * dim, seq, dim)
        ref.iris_dev_sync()
        theirs = lib.to_host(x, (seq, dim), np.float32)
        lib.check()
    finally:
        d.free()
    rel, cos_ = bc.delta_metrics(ours, theirs, inp["x"])
    assert rel <= 5e-3 and cos_ >= 0.99999, (rel, cos_)


# ---------------------------------------------------------------------------
# double-stream block
# ---------------------------------------------------------------------------

def device_double_block(lib, inp, key_mask=None):
    d = Dev(lib)
    try:
        dx = d.put(inp["x"])
        nbytes = lib.iris_b200_double_block_scratch_bytes(inp["seq"], inp["dim"], inp["mlp"])
        assert nbytes > 0
        scratch = d.new(nbytes)
        streams = [bc.StreamWeights(*[d.put(inp[s][k]) for k in bc.STREAM_KEYS]) for s in ("txt", "img")]
        dcos, dsin = d.put(inp["cos"]), d.put(inp["sin"])
        dm = d.put(np.ascontiguousarray(key_mask, np.int32)) if key_mask is not None else None
        rc = lib.iris_b200_double_block(dx, scratch, C.addressof(streams[0]), C.addressof(streams[1]), dcos, dsin,
                                        inp["seq"], inp["txt_seq"], inp["dim"], inp["heads"], inp["mlp"], dm)
        assert rc == 0
        out = lib.to_host(dx, inp["x"].shape, np.float32)
        lib.check()
        return out
    finally:
        d.free()


@pytest.mark.parametrize("case", [bc.SMALL, bc.MID, bc.KLEIN4B_SHORT], ids=lambda c: c["name"])
def test_double_block_against_the_restatement(lib, case):
    inp = bc.double_inputs(case)
    got = device_double_block(lib, inp)
    rel, cos = bc.delta_metrics(got, bc.oracle_double_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_double_block_against_the_recorded_reference(lib):
    import os
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.double_inputs(bc.SMALL)
    rel, cos = bc.delta_metrics(device_double_block(lib, inp), gold["double/" + bc.SMALL["name"]], inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_double_block_with_key_mask_and_no_text(lib):
    inp = bc.double_inputs(bc.MID)
    mask = np.ones(inp["seq"], np.int32)
    mask[3:25] = 0
    got = device_double_block(lib, inp, mask)
    rel, cos = bc.delta_metrics(got, bc.oracle_double_block(inp, mask), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)
    # a block whose text stream is empty is a block over the image rows alone
    case = dict(bc.SMALL, name="flux2-double-no-text", txt=0)
    inp = bc.double_inputs(case)
    rel, cos = bc.delta_metrics(device_double_block(lib, inp), bc.oracle_double_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_double_block_argument_checks(lib):
    d = Dev(lib)
    try:
        p = d.new(1 << 16)
        good = bc.StreamWeights(*[p] * 7)
        bad = bc.StreamWeights(p, p, None, p, p, p, p)
        a, b = C.addressof(good), C.addressof(bad)
        assert lib.iris_b200_double_block(p, p, a, b, p, p, 8, 4, 256, 2, 64, None) == 1      # a weight is missing
        assert lib.iris_b200_double_block(p, p, a, a, p, p, 8, 9, 256, 2, 64, None) == 1      # txt_seq > seq
        assert lib.iris_b200_double_block(p, p, a, a, p, p, 8, 4, 250, 2, 64, None) == 1      # dim != heads * 128
        assert lib.iris_b200_double_block(p, p, a, None, p, p, 8, 4, 256, 2, 64, None) == 1
        lib.iris_b200_clear_error()
    finally:
        d.free()


# ---------------------------------------------------------------------------
# the input projection with SwiGLU in its epilogue
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cin,heads,mlp", [(200, 256, 2, 384), (129, 512, 2, 200), (77, 256, 0, 136),
                                                (300, 384, 0, 1024), (260, 384, 3, 392), (70, 128, 1, 128)])
def test_linear_glu(lib, rows, cin, heads, mlp):
    """Q / K / V columns as iris_b200_linear_qk_norm_rope stores them, and
    silu(gate) * up for the gate | up rows of W, against the restatement of
    the reference's sequence linear_bf16 -> head_norm_rope x 2 -> swiglu."""
    o = ol.oracle()
    nq = 3 * heads * 128
    x = ol.to_bf16(ol.randn(rows + mlp, rows, cin))
    W = ol.to_bf16(ol.randn(cin + mlp, nq + 2 * mlp, cin) / np.float32(np.sqrt(cin)))
    wq = (1 + 0.1 * ol.randn(3, 128)).astype(np.float32)
    wk = (1 + 0.1 * ol.randn(4, 128)).astype(np.float32)
    ang = ol.randn(5, rows, 64)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    hf = np.zeros((rows, nq + 2 * mlp), np.float32)
    o.orc_linear(hf, nq + 2 * mlp, x, cin, W, cin, rows, cin, nq + 2 * mlp, 0)
    h = ol.to_bf16(hf)
    if heads:
        o.orc_head_norm_rope_bf16(h.ctypes.data, nq + 2 * mlp, wq, cos, sin, rows, heads, 128, 1e-6, 0)
        o.orc_head_norm_rope_bf16(h.ctypes.data + 2 * heads * 128, nq + 2 * mlp, wk, cos, sin, rows, heads, 128, 1e-6, 0)
    want_act = np.zeros((rows, mlp), np.uint16)
    o.orc_swiglu(want_act.ctypes.data, mlp, h.ctypes.data + 2 * nq, h.ctypes.data + 2 * (nq + mlp), nq + 2 * mlp, rows, mlp)
    lda = mlp + 16
    d = Dev(lib)
    try:
        dx, dW, dwq, dwk, dcos, dsin = (d.put(a) for a in (x, W, wq, wk, cos, sin))
        dqkv = d.put(np.full((rows, max(nq, 8)), 0x7FC0, np.uint16)) if heads else None
        dact = d.put(np.full((rows, lda), 0x7FC0, np.uint16))
        rc = lib.iris_b200_linear_glu(dqkv, nq, dact, lda, dx, dW, rows, cin, heads, mlp,
                                      dwq if heads else None, dwk if heads else None,
                                      dcos if heads else None, dsin if heads else None, 1e-6)
        assert rc == 0
        act = lib.to_host(dact, (rows, lda), np.uint16)
        qkv = lib.to_host(dqkv, (rows, nq), np.uint16) if heads else None
        lib.check()
    finally:
        d.free()
    assert (act[:, mlp:] == 0x7FC0).all()                     # nothing beyond the mlp columns is written
    fa, fw = ol.from_bf16(act[:, :mlp]), ol.from_bf16(want_act)
    assert np.isfinite(fa).all()
    # fp32 accumulation order differs from the restatement: a product on a bf16 rounding boundary may fall
    # either way, so allow two units in the last place of the larger of |value| and the operands' scale
    tol = np.maximum(np.abs(fw), 0.05) * 2.0 ** -6
    assert (np.abs(fa - fw) <= tol).all(), float(np.abs(fa - fw).max())
    assert (act[:, :mlp] != want_act).mean() < 0.1
    if heads:
        fq, fh = ol.from_bf16(qkv), ol.from_bf16(h[:, :nq])
        # two bf16 steps of the largest value of the (row, head): the rotation mixes a pair, so a product that
        # rounded the other way shows up in an element that may itself be small
        top = np.abs(fh).reshape(rows, 3 * heads, 128).max(axis=2, keepdims=True)
        tol = np.broadcast_to(np.maximum(top, 0.05) * 2.0 ** -6, (rows, 3 * heads, 128)).reshape(rows, nq)
        assert (np.abs(fq - fh) <= tol).all(), float(np.abs(fq - fh).max())
        assert (qkv != h[:, :nq]).mean() < 0.1


# ---------------------------------------------------------------------------
# FLUX.3 block: rows in segments with their own modulation
# ---------------------------------------------------------------------------

def device_f3_block(lib, inp, eps=1e-6, key_mask=None):
    d = Dev(lib)
    try:
        dx = d.put(inp["x"])
        scratch = d.new(lib.iris_b200_single_block_scratch_bytes(inp["seq"], inp["dim"], inp["mlp"]))
        args = [d.put(inp[k]) for k in ("w_in", "w_out", "norm_q", "norm_k")]
        n = len(inp["seg_mod"])
        segs = (bc.Segment * n)(*[bc.Segment(int(s), int(l), d.put(m))
                                  for s, l, m in zip(inp["seg_start"], inp["seg_len"], inp["seg_mod"])])
        dcos, dsin = d.put(inp["cos"]), d.put(inp["sin"])
        dm = d.put(np.ascontiguousarray(key_mask, np.int32)) if key_mask is not None else None
        rc = lib.iris_b200_single_block_segments(dx, scratch, *args, C.addressof(segs), n, dcos, dsin, inp["seq"],
                                                 inp["dim"], inp["heads"], inp["mlp"], eps, dm)
        assert rc == 0
        out = lib.to_host(dx, inp["x"].shape, np.float32)
        lib.check()
        return out
    finally:
        d.free()


@pytest.mark.parametrize("case", [bc.F3_SMALL, bc.F3_MID, bc.F3_KLEIN_SHORT], ids=lambda c: c["name"])
def test_f3_block_against_the_restatement(lib, case):
    """Segment boundaries fall inside 32-row groups and 128-row tiles (33, 133;
    40, 172; 64, 160): shift, scale and gate are picked per row."""
    inp = bc.f3_inputs(case)
    got = device_f3_block(lib, inp)
    rel, cos = bc.delta_metrics(got, bc.oracle_f3_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_f3_block_against_the_recorded_reference(lib):
    import os
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.f3_inputs(bc.F3_SMALL)
    rel, cos = bc.delta_metrics(device_f3_block(lib, inp)[::2], gold["f3/" + bc.F3_SMALL["name"]], inp["x"][::2])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_segments_must_tile_the_rows(lib):
    d = Dev(lib)
    try:
        p = d.new(1 << 16)
        gap = (bc.Segment * 2)(bc.Segment(0, 4, p), bc.Segment(5, 3, p))
        short = (bc.Segment * 1)(bc.Segment(0, 7, p))
        five = (bc.Segment * 5)(*[bc.Segment(i, 1, p) for i in range(5)])
        for segs, n in ((gap, 2), (short, 1), (five, 5)):
            assert lib.iris_b200_single_block_segments(p, p, p, p, p, p, C.addressof(segs), n, p, p, 8, 256, 2, 64,
                                                       1e-6, None) == 1
        lib.iris_b200_clear_error()
    finally:
        d.free()


# ---------------------------------------------------------------------------
# Z-Image block and its row operators
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("rows,dim", [(40, 3840), (9, 512), (5, 4100), (6, 1030)])
def test_rms_norm_rows(lib, rows, dim):
    o = ol.oracle()
    x, a = (ol.randn(rows, rows, dim) * 2).astype(np.float32), ol.randn(rows + 1, rows, dim)
    w, m = (1 + 0.1 * ol.randn(3, dim)).astype(np.float32), (0.5 * ol.randn(4, dim)).astype(np.float32)
    d = Dev(lib)
    try:
        dx, da, dw, dm, dout = d.put(x), d.put(a), d.put(w), d.put(m), d.new(rows * dim * 2)
        for scale, ps in ((m, dm), (None, None)):
            if scale is None:
                lib.iris_dev_rms_norm(dout, dx, dw, rows, dim, 1e-5)
            else:
                lib.iris_dev_rms_norm_mod(dout, dx, dw, ps, rows, dim, 1e-5)
            got = lib.to_host(dout, (rows, dim), np.uint16)
            lib.check()
            want = np.zeros((rows, dim), np.uint16)
            o.orc_rms_norm_mod(want, x, w, scale, rows, dim, 1e-5)
            fw = ol.from_bf16(want)
            assert (got != want).mean() < 0.02
            assert (np.abs(ol.from_bf16(got) - fw) <= bf16_ulp(fw) * 1.01).all()
        for gate, pg in ((m, dm), (None, None)):
            dy = d.put(x)
            lib.iris_dev_rms_norm_residual(dy, da, dw, pg, rows, dim, 1e-5)
            got = lib.to_host(dy, (rows, dim), np.float32)
            lib.check()
            want = x.copy()
            o.orc_rms_norm_residual(want, a, w, gate, rows, dim, 1e-5)
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    finally:
        d.free()


def device_zi_block(lib, inp):
    d = Dev(lib)
    try:
        dx = d.put(inp["x"])
        scratch = d.new(lib.iris_b200_zimage_block_scratch_bytes(inp["seq"], inp["dim"], inp["ff"]))
        w = bc.ZImageWeights(*[d.put(inp["w"][k]) for k in bc.ZI_KEYS])
        dmod = d.put(inp["mod"]) if inp["mod"] is not None else None
        dcos, dsin = d.put(inp["cos"]), d.put(inp["sin"])
        dm = d.put(np.ascontiguousarray(inp["mask"], np.int32)) if inp["mask"] is not None else None
        rc = lib.iris_b200_zimage_block(dx, scratch, C.addressof(w), dmod, dcos, dsin, inp["seq"], inp["dim"], inp["heads"],
                                        inp["ff"], dm)
        assert rc == 0
        out = lib.to_host(dx, inp["x"].shape, np.float32)
        lib.check()
        return out
    finally:
        d.free()


@pytest.mark.parametrize("case,modulated", [(bc.ZI_SMALL, True), (bc.ZI_SMALL, False), (bc.ZI_MID, True),
                                            (bc.ZI_30_HEADS, True)], ids=lambda v: v["name"] if isinstance(v, dict) else str(v))
def test_zimage_block_against_the_restatement(lib, case, modulated):
    inp = bc.zi_inputs(case, modulated=modulated)
    got = device_zi_block(lib, inp)
    rel, cos = bc.delta_metrics(got, bc.oracle_zi_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_zimage_block_against_the_recorded_reference(lib):
    import os
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.zi_inputs(bc.ZI_SMALL)
    rel, cos = bc.delta_metrics(device_zi_block(lib, inp)[::2], gold["zi/" + bc.ZI_SMALL["name"]], inp["x"][::2])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_zimage_block_argument_checks(lib):
    d = Dev(lib)
    try:
        p = d.new(1 << 16)
        good = bc.ZImageWeights(*[p] * 10)
        bad = bc.ZImageWeights(*([p] * 9 + [None]))
        assert lib.iris_b200_zimage_block(p, p, C.addressof(bad), p, p, p, 8, 256, 2, 64, None) == 1
        assert lib.iris_b200_zimage_block(p, p, C.addressof(good), p, p, p, 8, 250, 2, 64, None) == 1
        assert lib.iris_b200_zimage_block(p, p + 8, C.addressof(good), p, p, p, 8, 256, 2, 64, None) == 1
        assert lib.iris_b200_zimage_block_scratch_bytes(8, 256, 0) == 0
        lib.iris_b200_clear_error()
    finally:
        d.free()


# ---------------------------------------------------------------------------
# the linear layers as single CTAs (128 x 256 tiles) instead of the default
# CTA pairs (256 x 256 tiles, tcgen05.mma.cta_group::2)
# ---------------------------------------------------------------------------

@pytest.fixture
def pairs(lib):
    """The library with the other of its two GEMM kernels selected."""
    was = lib.iris_b200_linear_cta_pairs(0)
    assert was == 1                       # pairs are the default
    yield lib
    lib.iris_b200_linear_cta_pairs(was)
    lib.check()


@pytest.mark.parametrize("rows,cin,cout", [(200, 512, 264), (129, 1280, 512), (1, 64, 8), (700, 256, 1032)])
def test_single_ctas_linear_f32_and_residual(pairs, rows, cin, cout):
    test_linear_f32_and_linear_residual(pairs, rows, cin, cout)


@pytest.mark.parametrize("rows,cin,heads,mlp", [(200, 256, 2, 384), (129, 512, 2, 200), (77, 256, 0, 136), (300, 384, 0, 1024),
                                                (260, 384, 3, 392)])
def test_single_ctas_linear_glu(pairs, rows, cin, heads, mlp):
    test_linear_glu(pairs, rows, cin, heads, mlp)


def test_pairs_bf16_linear_matches_single_ctas(lib):
    """The plain bf16 GEMM on an odd number of row tiles and a partial column
    tile: identical bits from pairs and from single CTAs (same k order)."""
    rows, cin, cout = 900, 1024, 1160
    a = ol.to_bf16(ol.randn(1, rows, cin))
    W = ol.to_bf16(ol.randn(2, cout, cin) / np.float32(32.0))
    d = Dev(lib)
    try:
        da, dW, dy = d.put(a), d.put(W), d.new(rows * cout * 2)
        outs = []
        for mode in (0, 1):
            was = lib.iris_b200_linear_cta_pairs(mode)
            lib.iris_dev_linear_bf16(dy, da, dW, rows, cin, cout)
            outs.append(lib.to_host(dy, (rows, cout), np.uint16))
            lib.iris_b200_linear_cta_pairs(was)
            lib.check()
    finally:
        d.free()
    assert np.array_equal(outs[0], outs[1])
    want = ol.from_bf16(a).astype(np.float64) @ ol.from_bf16(W).astype(np.float64).T
    assert np.abs(ol.from_bf16(outs[1]) - want).max() <= 0.02 * np.abs(want).max()


@pytest.mark.parametrize("case", [bc.SMALL, bc.MID, bc.ODD_HEADS], ids=lambda c: c["name"])
def test_single_ctas_blocks(pairs, case):
    """Single, double (two row groups) and segmented blocks with every linear layer on single CTAs."""
    inp = bc.block_inputs(case)
    rel, cos = bc.delta_metrics(device_block(pairs, inp), bc.oracle_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)
    inp = bc.double_inputs(case)
    rel, cos = bc.delta_metrics(device_double_block(pairs, inp), bc.oracle_double_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)
    f3 = bc.F3_SMALL if case is bc.SMALL else bc.F3_MID
    inp = bc.f3_inputs(f3)
    rel, cos = bc.delta_metrics(device_f3_block(pairs, inp), bc.oracle_f3_block(inp), inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)
