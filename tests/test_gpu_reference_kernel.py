"""GPU against GPU: this library and the reference's own CUDA backend
(iris_cuda.cu compiled unmodified for sm_100, oracle/_ref) on the same device
buffers. The reference kernels use the same arithmetic rules (fp32 math, one
RNE rounding in the prologue; P rounded to bf16, fp32 row sum in attention),
so the prologue must agree to the last bit almost everywhere and the
attention far inside the parity gate."""
import numpy as np
import pytest

import oracle_lib as ol
import path_cases as pc

pytestmark = pytest.mark.gpu

D = 128


@pytest.fixture(scope="module")
def libs():
    import __graft_entry__ as ge
    ref = ol.ref_cuda()
    if ref is None:
        pytest.skip("oracle/_ref/libiris_ref_cuda.so not built")
    lib = ge.load_package().load()
    lib.init()
    assert ref.iris_dev_init() == 1
    yield lib, ref
    lib.check()


@pytest.mark.parametrize("case", [pc.FLUX_SMALL, pc.FLUX3_SMALL, pc.ZIMAGE_SMALL, pc.FLUX_CFG1],
                         ids=lambda c: c["name"])
def test_same_inputs_same_results_as_the_reference_kernels(libs, case):
    lib, ref = libs
    ours, theirs = pc.DeviceCase(lib, case), pc.DeviceCase(lib, case)
    try:
        ours.prologue(fused=True)
        ours.attention(kernel=0)
        lib.iris_dev_sync()
        for which in ("q", "k"):
            ref.iris_dev_head_norm_rope(theirs.ptr(which), theirs.ldi, theirs.w, theirs.cos, theirs.sin,
                                        theirs.seq, theirs.H, D, case["eps"], 0)
        ref.iris_dev_attention(theirs.out, theirs.hd, theirs.ptr("q"), theirs.ptr("k"), theirs.ptr("v"),
                               theirs.ldi, theirs.seq, theirs.seq, theirs.H, theirs.H, D,
                               1.0 / np.sqrt(D), 0, theirs.mask)
        ref.iris_dev_sync()
        a, b = ours.read_qkv(), theirs.read_qkv()
        oa, ob = ours.read_out(), theirs.read_out()
        lib.check()
    finally:
        ours.free()
        theirs.free()
    # prologue: identical bits except rare last-place differences (rsqrt / fma contraction)
    assert (a != b).mean() < 0.02
    fa, fb = ol.from_bf16(a), ol.from_bf16(b)
    assert (np.abs(fa - fb) <= np.maximum(np.abs(fb), 2.0 ** -6) * 2.0 ** -7).all()
    # attention: bf16 output against bf16 output
    mx, cs = ol.compare_heads(oa, ob, case["heads"])
    assert mx.max() <= 1e-2 and cs.min() >= 0.99995, (mx, cs)
