"""Pins the CPU restatement (oracle/iris_oracle.c): against golden vectors
recorded from the reference's own CPU code (tests/golden/reference_cpu.npz),
and, where the compiled reference is at hand (oracle/_ref), against it
directly on fresh inputs."""
import numpy as np
import pytest

import oracle_lib as ol

H, D = 2, 128
ATOL = 2e-5      # fp32 sums in another order + -ffast-math in the reference build


def close(a, b, atol=ATOL):
    np.testing.assert_allclose(a, b, rtol=0, atol=atol)


def test_generator_matches_reference(golden):
    o = ol.oracle()
    o.orc_rng_seed(42)
    u = np.array([o.orc_random_uniform() for _ in range(16)], np.float32)
    assert np.array_equal(u, golden["rng_uniform_seed42"])
    close(ol.randn(42, 64), golden["rng_normal_seed42"], 1e-6)
    close(ol.randn(1000, 64), golden["rng_normal_seed1000"], 1e-6)


def test_bf16_rounding_rule():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.1415927, 1e-30, 65504.0], np.float32)
    bits = ol.to_bf16(x)
    u = x.view(np.uint32).astype(np.uint64)
    want = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(bits, want)
    # ties go to the even mantissa
    assert ol.to_bf16(np.array([1.00390625], np.float32))[0] == 0x3F80
    assert ol.to_bf16(np.array([1.01171875], np.float32))[0] == 0x3F82
    assert np.array_equal(ol.to_bf16(ol.from_bf16(bits)), bits)


def test_fast_exp_error_bound():
    o = ol.oracle()
    xs = np.linspace(-80, 80, 4001)
    got = np.array([o.orc_fast_expf(float(x)) for x in xs])
    rel = np.abs(got - np.exp(xs)) / np.exp(xs)
    assert rel.max() < 1e-5
    assert o.orc_fast_expf(-100.0) == 0.0


def test_softmax(golden):
    o = ol.oracle()
    x = ol.randn(7, 5, 37) * np.float32(3.0)
    o.orc_softmax(x.reshape(-1), 5, 37)
    close(x, golden["softmax_seed7_5x37"], 1e-6)
    close(x.sum(1), np.ones(5), 1e-5)


def test_flash_attention_tiled_and_small(golden):
    o = ol.oracle()
    Hh = 3
    q, k, v = ol.randn(11, 70, Hh * D), ol.randn(12, 150, Hh * D), ol.randn(13, 150, Hh * D)
    out = np.zeros_like(q)
    o.orc_flash_attention(out, q, k, v, 70, 150, Hh, D, 1 / np.sqrt(D))
    close(out, golden["flash_tiled_70x150_h3"])
    out = np.zeros((40, Hh * D), np.float32)
    o.orc_flash_attention(out, q[:40].copy(), k[:100].copy(), v[:100].copy(), 40, 100, Hh, D, 1 / np.sqrt(D))
    close(out, golden["flash_small_40x100_h3"])
    # the strided device-surface oracle computes the same function
    close(ol.dev_attention(q[:40], k[:100], v[:100], Hh), golden["flash_small_40x100_h3"])


def test_naive_attention(golden):
    o = ol.oracle()
    B, Hh, Sq, Sk, Dd = 2, 2, 9, 21, 64
    q, k, v = ol.randn(21, B, Hh, Sq, Dd), ol.randn(22, B, Hh, Sk, Dd), ol.randn(23, B, Hh, Sk, Dd)
    out = np.zeros_like(q)
    o.orc_attention(out.reshape(-1), q.reshape(-1), k.reshape(-1), v.reshape(-1), B, Hh, Sq, Sk, Dd, 0.125)
    close(out, golden["attention_b2h2_9x21_d64"])


def test_legacy_rope(golden):
    o = ol.oracle()
    pos = np.arange(0, 33, 3, dtype=np.int32)
    fr = np.zeros((pos.size, 32, 2), np.float32)
    o.orc_compute_rope_freqs(fr.reshape(-1), pos, pos.size, 64, 10000.0)
    close(fr, golden["rope_freqs_dim64_theta1e4"], 1e-6)
    x = ol.randn(31, 2, pos.size, 3, 64)
    o.orc_apply_rope(x.reshape(-1), golden["rope_freqs_dim64_theta1e4"].reshape(-1), 2, pos.size, 3, 64)
    close(x, golden["apply_rope_split_half"], 1e-6)


def flux_tables(txt, ph, pw, t_offset=0):
    o = ol.oracle()
    ct = np.zeros((txt, 64), np.float32); st = np.zeros_like(ct)
    o.orc_flux_rope_text(ct, st, txt, 32, 2000.0)
    ci = np.zeros((ph * pw, 64), np.float32); si = np.zeros_like(ci)
    o.orc_flux_rope_image(ci, si, ph, pw, 32, 2000.0, t_offset)
    return ct, st, ci, si


def test_flux_tables(golden):
    ct, st, ci, si = flux_tables(24, 4, 6)
    close(ct, golden["flux_rope_text_cos"], 1e-6); close(st, golden["flux_rope_text_sin"], 1e-6)
    close(ci, golden["flux_rope_img_cos"], 1e-6); close(si, golden["flux_rope_img_sin"], 1e-6)
    _, _, cr, sr = flux_tables(1, 4, 6, 10)
    close(cr, golden["flux_rope_ref10_cos"], 1e-6); close(sr, golden["flux_rope_ref10_sin"], 1e-6)


def test_rope_convention_against_published_formula():
    """Token at (T, H, W, L) = (10, 5, 3, 0), theta 2000: the table and pair
    rotation must equal the rotation-matrix form [[cos, -sin], [sin, cos]]
    with omega_d = theta^(-2d/32) per axis (the check of the reference's
    debug/debug_rope_img2img.py)."""
    o = ol.oracle()
    c = np.zeros((6 * 4, 64), np.float32); s = np.zeros_like(c)
    o.orc_flux_rope_image(c, s, 6, 4, 32, 2000.0, 10)
    row = 5 * 4 + 3
    omega = 1.0 / (2000.0 ** (np.arange(0, 32, 2) / 32.0))
    ang = np.concatenate([p * omega for p in (10, 5, 3, 0)])
    close(c[row], np.cos(ang), 2e-6); close(s[row], np.sin(ang), 2e-6)
    x = ol.randn(123, 1, 128)
    y = x.copy()
    ones = np.ones(128, np.float32)
    # eps chosen so that the norm factor is exactly recoverable
    o.orc_head_norm_rope_f32(y.ctypes.data, 128, ones, c[row:row + 1].copy(), s[row:row + 1].copy(), 1, 1, 128, 1e-6, 0)
    xn = x[0] / np.sqrt((x[0].astype(np.float64) ** 2).mean() + 1e-6)
    pairs = xn.reshape(64, 2)
    want = np.stack([np.cos(ang) * pairs[:, 0] - np.sin(ang) * pairs[:, 1],
                     np.sin(ang) * pairs[:, 0] + np.cos(ang) * pairs[:, 1]], 1).reshape(-1)
    close(y[0], want, 1e-5)


def flux_inputs():
    txt, img = 24, 24
    t = [ol.randn(1000 + i, txt, H * D) for i in range(3)]
    im = [ol.randn(42 + i, img, H * D) for i in range(3)]
    return [np.concatenate([a, b]) for a, b in zip(t, im)]


def test_flux_prologue_and_attention(golden):
    o = ol.oracle()
    q, k, v = flux_inputs()
    ct, st, ci, si = flux_tables(24, 4, 6)
    cos, sin = np.concatenate([ct, ci]), np.concatenate([st, si])
    o.orc_head_norm_rope_f32(q.ctypes.data, H * D, golden["flux_wq"], cos, sin, 48, H, D, 1e-6, 0)
    o.orc_head_norm_rope_f32(k.ctypes.data, H * D, golden["flux_wk"], cos, sin, 48, H, D, 1e-6, 0)
    close(q, golden["flux_q_prologue"]); close(k, golden["flux_k_prologue"])
    out = ol.dev_attention(q, k, v, H)
    close(out, golden["flux_joint_out"])       # joint attention over [TEXT, IMAGE]
    close(out, golden["flux_single_out"])      # == self attention of the concatenation


def test_flux3_prologue_and_attention(golden):
    o = ol.oracle()
    rh = np.array([4, 2], np.int32); rw = np.array([4, 6], np.int32)
    total = 16 + 16 + 16 + 12
    c = np.zeros((total, 64), np.float32); s = np.zeros_like(c)
    assert o.orc_f3_joint_rope(c, s, 16, 4, 4, rh, rw, 2, D, 10000.0) == total
    close(c, golden["f3_rope_cos"], 1e-6); close(s, golden["f3_rope_sin"], 1e-6)
    q, k, v = (ol.randn(2000 + i, total, H * D) for i in range(3))
    o.orc_head_norm_rope_f32(q.ctypes.data, H * D, golden["flux_wq"], c, s, total, H, D, 1e-6, 0)
    o.orc_head_norm_rope_f32(k.ctypes.data, H * D, golden["flux_wk"], c, s, total, H, D, 1e-6, 0)
    close(q, golden["f3_q_prologue"]); close(k, golden["f3_k_prologue"])
    close(ol.dev_attention(q, k, v, H), golden["f3_out"])


def test_zimage_prologue_and_masked_attention(golden):
    o = ol.oracle()
    pos = np.zeros((64, 3), np.int32); mask = np.zeros(64, np.int32)
    assert o.orc_zi_positions(pos.reshape(-1), mask, 5, 6, 20) == 64
    assert np.array_equal(pos, golden["zi_pos"]) and np.array_equal(mask, golden["zi_mask"])
    assert mask.sum() == 50 and pos[0, 0] == 33 and pos[32, 0] == 1
    c = np.zeros((64, 64), np.float32); s = np.zeros_like(c)
    o.orc_zi_rope(c, s, pos.reshape(-1), 64, 256.0)
    x = ol.randn(3000, 64, H * D)
    q = x.copy()
    ones = np.ones(D, np.float32)
    o.orc_head_norm_rope_f32(q.ctypes.data, H * D, ones, c, s, 64, H, D, 1e-5, 0)
    close(q, golden["zi_q_prologue"])
    close(ol.dev_attention(q, q, x, H, key_mask=mask), golden["zi_masked_out"])
    close(ol.dev_attention(q, q, x, H), golden["zi_unmasked_out"])


def test_dev_attention_semantics():
    """GQA, causal limit, sampled rows and the all-masked row of the device op."""
    q, k, v = ol.randn(1, 12, 4 * 64), ol.randn(2, 20, 2 * 64), ol.randn(3, 20, 2 * 64)
    full = ol.dev_attention(q, k, v, 4, kv_heads=2, head_dim=64)
    # query head h reads kv head h // 2
    for h in range(4):
        one = ol.dev_attention(q[:, h * 64:(h + 1) * 64], k[:, (h // 2) * 64:(h // 2 + 1) * 64],
                               v[:, (h // 2) * 64:(h // 2 + 1) * 64], 1, head_dim=64)
        close(full[:, h * 64:(h + 1) * 64], one, 1e-6)
    ca = ol.dev_attention(q, k, v, 4, kv_heads=2, head_dim=64, causal=1)
    close(ca[0, :64], v[0, :64], 1e-6)          # query 0 sees key 0 only
    rows = np.array([3, 7], np.int32)
    part = ol.dev_attention(q, k, v, 4, kv_heads=2, head_dim=64, rows=rows)
    close(part[rows], full[rows], 0)
    assert not part[0].any()
    none = ol.dev_attention(q, k, v, 4, kv_heads=2, head_dim=64, key_mask=np.zeros(20, np.int32))
    assert not none.any()
    mx, cs = ol.compare_heads(full, full, 4, 64)
    assert mx.max() == 0 and cs.min() > 0.999999


def test_bf16_prologue_rounds_once():
    o = ol.oracle()
    x = ol.randn(5, 6, 2 * 128)
    c, s = np.cos(ol.randn(6, 6, 64)), np.sin(ol.randn(6, 6, 64))
    c, s = np.ascontiguousarray(c, np.float32), np.ascontiguousarray(s, np.float32)
    w = np.ones(128, np.float32)
    xb = ol.to_bf16(x)
    xf = ol.from_bf16(xb)
    o.orc_head_norm_rope_f32(xf.ctypes.data, 256, w, c, s, 6, 2, 128, 1e-6, 1)
    o.orc_head_norm_rope_bf16(xb.ctypes.data, 256, w, c, s, 6, 2, 128, 1e-6, 1)
    assert np.array_equal(xb, ol.to_bf16(xf))


# ---------------------------------------------------------------------------
# Direct comparison with the compiled reference, where it is at hand.
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("kind", ["generic", "blas"])
def test_against_compiled_reference(kind):
    r = ol.ref(kind)
    if r is None:
        pytest.skip("oracle/_ref/libiris_ref_%s.so not built here" % kind)
    o = ol.oracle()
    if kind == "blas":
        r.openblas_set_num_threads(1)
    Hh, txt, ph, pw = 4, 40, 7, 9
    img = ph * pw
    seq = txt + img
    q, k, v = (ol.randn(500 + i, seq, Hh * D) for i in range(3))
    w = np.ones(D, np.float32)
    ct = np.zeros((txt, D), np.float32); st = np.zeros_like(ct)
    ci = np.zeros((img, D), np.float32); si = np.zeros_like(ci)
    r.ref_flux_rope_text(ct, st, txt, 32, 2000.0)
    r.ref_flux_rope_2d(ci, si, ph, pw, 32, 2000.0)
    rq, rk = q.copy(), k.copy()
    r.ref_flux_qk_norm(rq, rk, w, w, seq, Hh, D, 1e-6)
    for x in (rq, rk):
        r.ref_flux_apply_rope_2d(x[:txt], ct, st, txt, Hh, D)
        r.ref_flux_apply_rope_2d(x[txt:], ci, si, img, Hh, D)
    oct_, ost, oci, osi = flux_tables(txt, ph, pw)
    cos, sin = np.concatenate([oct_, oci]), np.concatenate([ost, osi])
    oq, ok = q.copy(), k.copy()
    o.orc_head_norm_rope_f32(oq.ctypes.data, Hh * D, w, cos, sin, seq, Hh, D, 1e-6, 0)
    o.orc_head_norm_rope_f32(ok.ctypes.data, Hh * D, w, cos, sin, seq, Hh, D, 1e-6, 0)
    close(oq, rq); close(ok, rk)
    io = np.zeros((img, Hh * D), np.float32); to = np.zeros((txt, Hh * D), np.float32)
    c = np.ascontiguousarray
    assert r.ref_flux_joint_attention(io, to, c(rq[txt:]), c(rk[txt:]), c(v[txt:]),
                                      c(rq[:txt]), c(rk[:txt]), c(v[:txt]), img, txt, Hh, D) == 0
    close(ol.dev_attention(oq, ok, v, Hh), np.concatenate([to, io]))
    o3 = np.zeros_like(q)
    assert r.ref_f3_attention(o3, rq, rk, v, seq, Hh, D) == 0
    close(ol.dev_attention(oq, ok, v, Hh), o3)
