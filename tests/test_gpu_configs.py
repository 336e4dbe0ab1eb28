"""The five benchmark configurations at full size on the tcgen05 kernel:
parity on sampled query rows against the oracle (all heads), and
size-independent properties of attention that need no oracle."""
import numpy as np
import pytest

import oracle_lib as ol
import path_cases as pc

pytestmark = pytest.mark.gpu

D = 128
MAX_ABS, MIN_COS = 2e-2, 0.9999
TC = 1


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.check()


CONFIGS = [pc.FLUX_CFG1, pc.FLUX_CFG2, pc.FLUX_CFG3, pc.ZIMAGE_CFG4, pc.FLUX3_CFG5]


@pytest.mark.parametrize("case", CONFIGS, ids=lambda c: c["name"])
def test_config_parity(lib, case):
    for b in range(case.get("batch", 1)):
        res = pc.run_case(lib, case, kernel=TC, b=b)
        assert res["max_abs"] <= MAX_ABS and res["min_cos"] >= MIN_COS, (b, res["max_abs"], res["min_cos"])
        assert res["prologue_max_abs"] <= 11.4 * 2.0 ** -8


def test_klein4b_1024_every_row_against_the_reference_cpu_build(lib):
    """The headline configuration, all 4608 rows of all 24 heads, against the
    reference's own CPU code (its BLAS build compiled from its sources:
    qk_norm, its own RoPE tables and rotation, mha_forward) fed the same
    bf16-rounded inputs. Skipped where that build is absent."""
    r = ol.ref("blas") or ol.ref("generic")
    if r is None:
        pytest.skip("oracle/_ref is not built here")
    case = pc.FLUX_CFG2
    H, txt, (ih, iw) = case["heads"], case["txt"], case["img"]
    img, seq = ih * iw, pc.seq_len(case)
    dc = pc.DeviceCase(lib, case)
    try:
        dc.prologue(True)
        dc.attention(TC)
        got = dc.read_out()
        lib.check()
    finally:
        dc.free()
    q, k, v = pc.qkv_inputs(case)
    o = ol.oracle()
    for x in (q, k, v):
        o.orc_round_bf16(x.reshape(-1), x.size)
    w = np.ones(D, np.float32)
    ct = np.zeros((txt, D), np.float32); st = np.zeros_like(ct)
    ci = np.zeros((img, D), np.float32); si = np.zeros_like(ci)
    r.ref_flux_rope_text(ct, st, txt, 32, 2000.0)
    r.ref_flux_rope_2d(ci, si, ih, iw, 32, 2000.0)
    r.ref_flux_qk_norm(q, k, w, w, seq, H, D, case["eps"])
    for x in (q, k):
        r.ref_flux_apply_rope_2d(x[:txt], ct, st, txt, H, D)
        r.ref_flux_apply_rope_2d(x[txt:], ci, si, img, H, D)
    want = np.zeros_like(q)
    if hasattr(r, "openblas_set_num_threads"):
        r.openblas_set_num_threads(1)
        assert r.ref_flux_mha(want, q, k, v, seq, H, D) == 0
    else:
        r.iris_flash_attention(want, q, k, v, seq, seq, H, D, 1.0 / np.sqrt(D))
    mx, cs = ol.compare_heads(got, want, H)
    assert mx.max() <= MAX_ABS and cs.min() >= MIN_COS, (mx, cs)


def test_cfg_batch_shares_image_rows():
    """cond / uncond differ in the text rows only (two forward passes over the
    same latent, iris_sample.c:698-712)."""
    small = dict(pc.FLUX_SMALL, batch=2)
    q0, _, _ = pc.qkv_inputs(small, 0)
    q1, _, _ = pc.qkv_inputs(small, 1)
    t = small["txt"]
    assert np.array_equal(q0[t:], q1[t:]) and not np.array_equal(q0[:t], q1[:t])


def test_auto_dispatch_matches_reference_rule(lib):
    """AUTO takes the tensor-core kernel exactly where the reference takes its
    flash kernel (iris_cuda.cu:884-886) and TMA can address the views."""
    f = lib.iris_b200_attention_kernel_for
    assert f(256, 3072, 256, 512, 768, 9216, 24, 24, 128, 0) == 1
    assert f(256, 3072, 256, 512, 768, 9216, 24, 24, 128, 1) == 2     # causal
    assert f(256, 3072, 256, 512, 768, 9216, 24, 8, 128, 0) == 2      # GQA
    assert f(256, 3072, 256, 512, 768, 9216, 24, 24, 64, 0) == 2      # head_dim
    assert f(256, 3072, 256, 512, 768, 9220, 24, 24, 128, 0) == 2     # ldi % 8
    assert f(256, 3072, 258, 512, 768, 9216, 24, 24, 128, 0) == 2     # alignment


def full_size_buffers(lib, seq, H, seed):
    hd = H * D
    q = ol.to_bf16(ol.randn(seed, seq, hd))
    k = ol.to_bf16(ol.randn(seed + 1, seq, hd))
    return q, k


def run_attn(lib, q, k, v, H):
    seq_q, seq_k = q.shape[0], k.shape[0]
    dq, dk, dv = lib.to_device(q), lib.to_device(k), lib.to_device(v)
    dout = lib.alloc(seq_q * H * D * 2)
    assert lib.iris_b200_attention_ex(dout, H * D, dq, dk, dv, H * D, seq_q, seq_k, H, H, D,
                                      1.0 / np.sqrt(D), 0, None, TC) == 0
    out = lib.to_host(dout, (seq_q, H * D), np.uint16)
    lib.check()
    for p in (dq, dk, dv, dout):
        lib.iris_dev_free(p)
    return out


def test_full_size_properties(lib):
    """At the size of the headline configuration (4608 tokens, 24 heads):
    (1) softmax rows sum to one: V = 1 gives exactly 1;
    (2) permuting the keys (K and V rows together) leaves the output
        unchanged up to summation order;
    (3) linearity in V: attn(V1 + V2) = attn(V1) + attn(V2)."""
    seq, H = 4608, 24
    q, k = full_size_buffers(lib, seq, H, 77)
    ones = np.full((seq, H * D), 0x3F80, np.uint16)
    out = ol.from_bf16(run_attn(lib, q, k, ones, H))
    assert np.abs(out - 1.0).max() <= 2.0 ** -7

    v = ol.to_bf16(ol.randn(80, seq, H * D))
    base = ol.from_bf16(run_attn(lib, q, k, v, H))
    perm = np.random.default_rng(0).permutation(seq)
    shuf = ol.from_bf16(run_attn(lib, q, np.ascontiguousarray(k[perm]), np.ascontiguousarray(v[perm]), H))
    mx, cs = ol.compare_heads(base, shuf, H)
    assert mx.max() <= 4e-3 and cs.min() >= 0.99999

    v1 = ol.randn(81, seq, H * D)
    v2 = ol.randn(82, seq, H * D)
    b1, b2 = ol.to_bf16(v1), ol.to_bf16(v2)
    bsum = ol.to_bf16(ol.from_bf16(b1) + ol.from_bf16(b2))
    o1 = ol.from_bf16(run_attn(lib, q, k, b1, H))
    o2 = ol.from_bf16(run_attn(lib, q, k, b2, H))
    os_ = ol.from_bf16(run_attn(lib, q, k, bsum, H))
    mx, cs = ol.compare_heads(os_, o1 + o2, H)
    assert mx.max() <= 1e-2 and cs.min() >= 0.9999


def test_long_sequence_properties(lib):
    """16896 tokens (the multi-reference configuration): row sums and the
    invariance to a key rotation by a non-multiple of the tile size."""
    seq, H = 16896, 4
    q, k = full_size_buffers(lib, seq, H, 91)
    ones = np.full((seq, H * D), 0x3F80, np.uint16)
    out = ol.from_bf16(run_attn(lib, q, k, ones, H))
    assert np.abs(out - 1.0).max() <= 2.0 ** -7
    v = ol.to_bf16(ol.randn(93, seq, H * D))
    base = ol.from_bf16(run_attn(lib, q, k, v, H))
    rolled = ol.from_bf16(run_attn(lib, q, np.roll(k, 1000, axis=0).copy(), np.roll(v, 1000, axis=0).copy(), H))
    mx, cs = ol.compare_heads(base, rolled, H)
    assert mx.max() <= 4e-3 and cs.min() >= 0.99999
