"""CPU tests of the restatement of the operators around the attention path and
of one single-stream block: against numpy in float64, against the committed
outputs of the reference's CPU block, and against the reference itself where
oracle/_ref is built."""
import os
import sys

import numpy as np
import pytest

import block_cases as bc
import oracle_lib as ol

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_block_golden as mg  # noqa: E402

# The block's tolerance is the path's: what the bf16 intermediates of the
# device sequence cost against the reference's fp32 CPU block.
REL_MAX, MIN_COS = 2e-2, 0.9999


def bf16_ulp(x):
    return np.maximum(np.abs(x), 2.0 ** -126) * 2.0 ** -7


def test_layer_norm_mod_against_float64():
    o = ol.oracle()
    rows, dim = 9, 384
    x = ol.randn(3, rows, dim) * 3 + 1
    shift, scale = ol.randn(4, dim), ol.randn(5, dim) * np.float32(0.3)
    x64 = x.astype(np.float64)
    n = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-6)
    for sh, sc in ((shift, scale), (None, scale), (shift, None), (None, None)):
        out = np.zeros((rows, dim), np.uint16)
        o.orc_layer_norm_mod(out, x, sh, sc, rows, dim, 1e-6)
        want = n * (1 + (sc if sc is not None else 0)) + (sh if sh is not None else 0)
        assert (np.abs(ol.from_bf16(out) - want) <= bf16_ulp(want)).all()


def test_swiglu_and_residual_against_float64():
    o = ol.oracle()
    rows, cols, ldi, ldo = 7, 40, 100, 56
    src = ol.to_bf16(ol.randn(6, rows, ldi) * 4)
    out = np.zeros((rows, ldo), np.uint16)
    o.orc_swiglu(out.ctypes.data, ldo, src.ctypes.data, src.ctypes.data + 2 * 50, ldi, rows, cols)
    g, u = ol.from_bf16(src[:, :cols]).astype(np.float64), ol.from_bf16(src[:, 50:50 + cols]).astype(np.float64)
    want = g / (1 + np.exp(-g)) * u
    assert (np.abs(ol.from_bf16(out[:, :cols]) - want) <= bf16_ulp(want)).all()
    assert not out[:, cols:].any()
    x, a, gate = ol.randn(7, rows, cols), ol.randn(8, rows, cols), ol.randn(9, cols)
    x1, x2 = x.copy(), x.copy()
    o.orc_residual(x1, a, gate, rows, cols)
    o.orc_residual(x2, a, None, rows, cols)
    np.testing.assert_allclose(x1, x + gate * a, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(x2, x + a, rtol=1e-6, atol=1e-6)


def test_linear_against_float64():
    o = ol.oracle()
    rows, cin, cout = 13, 200, 24
    x, W = ol.to_bf16(ol.randn(10, rows, cin + 8)), ol.to_bf16(ol.randn(11, cout, cin))
    y = np.zeros((rows, cout + 3), np.float32)
    for threads in (1, 4):
        o.orc_linear(y, cout + 3, x, cin + 8, W, cin, rows, cin, cout, threads)
        want = ol.from_bf16(x[:, :cin]).astype(np.float64) @ ol.from_bf16(W).astype(np.float64).T
        np.testing.assert_allclose(y[:, :cout], want, rtol=1e-4, atol=1e-4)
        assert not y[:, cout:].any()


@pytest.mark.parametrize("case", [bc.SMALL, bc.MID], ids=lambda c: c["name"])
def test_block_restatement_against_recorded_reference(case):
    """The committed outputs of the reference's single_block_forward pin the
    restatement on machines without the reference sources."""
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.block_inputs(case)
    assert np.isclose(inp["x"].astype(np.float64).sum(), gold[case["name"] + "/x_sum"])
    step = mg.ROW_STEP[case["name"]]
    got = bc.oracle_block(inp)[::step]
    rel, cos = bc.delta_metrics(got, gold[case["name"]], inp["x"][::step])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_block_restatement_against_reference_build():
    r = ol.ref("generic")
    if r is None:
        pytest.skip("oracle/_ref is not built here")
    case = dict(bc.SMALL, name="flux2-block-other", txt=24, img=(6, 10))
    inp = bc.block_inputs(case, seed=31)
    want = mg.reference_block(r, case, inp)
    rel, cos = bc.delta_metrics(bc.oracle_block(inp), want, inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_key_mask_reaches_the_block():
    """Masked keys change the result, and a mask of ones does not."""
    inp = bc.block_inputs(bc.SMALL)
    base = bc.oracle_block(inp)
    ones = np.ones(inp["seq"], np.int32)
    assert np.array_equal(bc.oracle_block(inp, ones), base)
    m = ones.copy()
    m[5:20] = 0
    assert not np.array_equal(bc.oracle_block(inp, m), base)


def test_double_block_restatement_against_recorded_reference():
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.double_inputs(bc.SMALL)
    rel, cos = bc.delta_metrics(bc.oracle_double_block(inp), gold["double/" + bc.SMALL["name"]], inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_double_block_restatement_against_reference_build():
    r = ol.ref("generic")
    if r is None:
        pytest.skip("oracle/_ref is not built here")
    case = dict(bc.MID, name="flux2-double-other", txt=17, img=(7, 9))
    inp = bc.double_inputs(case, seed=41)
    want = mg.reference_double_block(r, case, inp)
    rel, cos = bc.delta_metrics(bc.oracle_double_block(inp), want, inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_double_block_streams_use_their_own_weights():
    """Swapping the two streams' weights changes the result: no stream is read twice."""
    inp = bc.double_inputs(bc.SMALL)
    base = bc.oracle_double_block(inp)
    swapped = bc.oracle_double_block(dict(inp, txt=inp["img"], img=inp["txt"]))
    assert not np.allclose(base, swapped)


def test_f3_block_restatement_against_recorded_reference():
    """FLUX.3: one block over text, image and reference-image segments with
    their own modulation, against the recorded output of the reference's
    block_forward (iris_transformer_flux3.c:371-417)."""
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.f3_inputs(bc.F3_SMALL)
    assert len(inp["seg_mod"]) == 3
    rel, cos = bc.delta_metrics(bc.oracle_f3_block(inp)[::2], gold["f3/" + bc.F3_SMALL["name"]], inp["x"][::2])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_f3_block_restatement_against_reference_build():
    r = ol.ref("generic")
    if r is None:
        pytest.skip("oracle/_ref is not built here")
    inp = bc.f3_inputs(bc.F3_MID, seed=77)
    want = mg.reference_f3_block(r, bc.F3_MID, inp)
    rel, cos = bc.delta_metrics(bc.oracle_f3_block(inp), want, inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_one_segment_is_the_single_block():
    inp = bc.block_inputs(bc.SMALL)
    seg = dict(inp, seg_start=np.array([0], np.int32), seg_len=np.array([inp["seq"]], np.int32), seg_mod=[inp["mod"]])
    assert np.array_equal(bc.oracle_f3_block(seg), bc.oracle_block(inp))


def test_rms_norm_rows_against_float64():
    o = ol.oracle()
    rows, dim = 7, 200
    x, a = ol.randn(1, rows, dim) * 2, ol.randn(2, rows, dim)
    w, m = (1 + 0.1 * ol.randn(3, dim)).astype(np.float32), (0.5 * ol.randn(4, dim)).astype(np.float32)
    x64 = x.astype(np.float64)
    n = x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-5) * w
    for scale in (m, None):
        out = np.zeros((rows, dim), np.uint16)
        o.orc_rms_norm_mod(out, x, w, scale, rows, dim, 1e-5)
        want = n * (1 + scale) if scale is not None else n
        assert (np.abs(ol.from_bf16(out) - want) <= bf16_ulp(want)).all()
    a64 = a.astype(np.float64)
    na = a64 / np.sqrt((a64 ** 2).mean(1, keepdims=True) + 1e-5) * w
    for gate in (m, None):
        y = x.copy()
        o.orc_rms_norm_residual(y, a, w, gate, rows, dim, 1e-5)
        np.testing.assert_allclose(y, x64 + (np.tanh(gate) if gate is not None else 1.0) * na, rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("modulated", [True, False], ids=["modulated", "context-refiner"])
def test_zimage_block_restatement_against_reference_build(modulated):
    r = ol.ref("generic")
    if r is None:
        pytest.skip("oracle/_ref is not built here")
    inp = bc.zi_inputs(bc.ZI_MID, seed=123, modulated=modulated)
    want = mg.reference_zi_block(r, bc.ZI_MID, inp)
    rel, cos = bc.delta_metrics(bc.oracle_zi_block(inp), want, inp["x"])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)


def test_zimage_block_restatement_against_recorded_reference():
    """One Z-Image block with padded image and caption rows under the key
    mask, against the recorded output of zi_block_forward
    (iris_transformer_zimage.c:801-880)."""
    gold = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block.npz")))
    inp = bc.zi_inputs(bc.ZI_SMALL)
    assert inp["mask"] is not None and not inp["mask"].all()
    rel, cos = bc.delta_metrics(bc.oracle_zi_block(inp)[::2], gold["zi/" + bc.ZI_SMALL["name"]], inp["x"][::2])
    assert rel <= REL_MAX and cos >= MIN_COS, (rel, cos)
