#!/usr/bin/env python3
"""Generate tests/golden/*.npz from the reference's own CPU code.

Run where the reference sources are present:

    make -C oracle ref && python tests/golden/make_golden.py

It loads oracle/_ref/libiris_ref_generic.so (the reference's iris_kernels.c
and the static helpers of its three transformer files, compiled unmodified
with the flags of `make generic`) and records, for small seeded inputs, the
outputs of every reference function on the joint-attention path. The
committed .npz files are what pins the CPU restatement in oracle/ on
machines where the reference sources are absent.

Inputs are not stored: they are regenerated from the seed with the
restatement's generator, which test_oracle.py first checks against the
recorded generator output.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402


def ref_randn(r, seed, *shape):
    out = np.empty(shape, np.float32)
    r.iris_rng_seed(seed)
    r.iris_randn(out.reshape(-1), out.size)
    return out


def expand_pairs(t):
    """[seq, hd/2] -> [seq, hd] with each value duplicated for its pair."""
    return np.ascontiguousarray(np.repeat(t, 2, axis=1))


def main():
    r = ol.ref("generic")
    if r is None:
        sys.exit("oracle/_ref/libiris_ref_generic.so missing: run `make -C oracle ref` first")
    g = {}

    # --- generator -------------------------------------------------------
    r.iris_rng_seed(42)
    g["rng_uniform_seed42"] = np.array([r.iris_random_uniform() for _ in range(16)], np.float32)
    g["rng_normal_seed42"] = ref_randn(r, 42, 64)
    g["rng_normal_seed1000"] = ref_randn(r, 1000, 64)

    # --- iris_kernels.h surface -------------------------------------------
    x = ref_randn(r, 7, 5, 37) * 3.0
    sm = x.copy()
    r.iris_softmax(sm.reshape(-1), 5, 37)
    g["softmax_seed7_5x37"] = sm

    H, D = 3, 128
    q = ref_randn(r, 11, 70, H * D)
    k = ref_randn(r, 12, 150, H * D)
    v = ref_randn(r, 13, 150, H * D)
    out = np.zeros_like(q)
    r.iris_flash_attention(out, q, k, v, 70, 150, H, D, 1.0 / np.sqrt(D))
    g["flash_tiled_70x150_h3"] = out
    out = np.zeros((40, H * D), np.float32)
    r.iris_flash_attention(out, q[:40].copy(), k[:100].copy(), v[:100].copy(), 40, 100, H, D, 1.0 / np.sqrt(D))
    g["flash_small_40x100_h3"] = out

    B, Hh, Sq, Sk, Dd = 2, 2, 9, 21, 64
    q = ref_randn(r, 21, B, Hh, Sq, Dd)
    k = ref_randn(r, 22, B, Hh, Sk, Dd)
    v = ref_randn(r, 23, B, Hh, Sk, Dd)
    out = np.zeros_like(q)
    r.iris_attention(out.reshape(-1), q.reshape(-1), k.reshape(-1), v.reshape(-1), B, Hh, Sq, Sk, Dd, 0.125)
    g["attention_b2h2_9x21_d64"] = out

    pos = np.arange(0, 33, 3, dtype=np.int32)
    fr = np.zeros((pos.size, 32, 2), np.float32)
    r.iris_compute_rope_freqs(fr.reshape(-1), pos, pos.size, 64, 10000.0)
    g["rope_freqs_dim64_theta1e4"] = fr
    x = ref_randn(r, 31, 2, pos.size, 3, 64)
    r.iris_apply_rope(x.reshape(-1), fr.reshape(-1), 2, pos.size, 3, 64)
    g["apply_rope_split_half"] = x

    # --- FLUX.2: tables, prologue, joint attention -------------------------
    txt, ph, pw, H, D = 24, 4, 6, 2, 128
    img = ph * pw
    ct = np.zeros((txt, D), np.float32); st = np.zeros_like(ct)
    r.ref_flux_rope_text(ct, st, txt, 32, 2000.0)
    ci = np.zeros((img, D), np.float32); si = np.zeros_like(ci)
    r.ref_flux_rope_2d(ci, si, ph, pw, 32, 2000.0)
    cr = np.zeros((img, D), np.float32); sr = np.zeros_like(cr)
    r.ref_flux_rope_2d_t(cr, sr, ph, pw, 32, 2000.0, 10)
    g["flux_rope_text_cos"], g["flux_rope_text_sin"] = ct[:, ::2].copy(), st[:, ::2].copy()
    g["flux_rope_img_cos"], g["flux_rope_img_sin"] = ci[:, ::2].copy(), si[:, ::2].copy()
    g["flux_rope_ref10_cos"], g["flux_rope_ref10_sin"] = cr[:, ::2].copy(), sr[:, ::2].copy()
    assert np.array_equal(ct[:, ::2], ct[:, 1::2]) and np.array_equal(si[:, ::2], si[:, 1::2])

    w_q = 1.0 + 0.1 * ref_randn(r, 41, D)
    w_k = 1.0 + 0.1 * ref_randn(r, 42, D)
    g["flux_wq"], g["flux_wk"] = w_q, w_k
    tq, tk, tv = (ref_randn(r, 1000 + i, txt, H * D) for i in range(3))
    iq, ik, iv = (ref_randn(r, 42 + i, img, H * D) for i in range(3))
    r.ref_flux_qk_norm(tq, tk, w_q, w_k, txt, H, D, 1e-6)
    r.ref_flux_qk_norm(iq, ik, w_q, w_k, img, H, D, 1e-6)
    r.ref_flux_apply_rope_2d(tq, ct, st, txt, H, D)
    r.ref_flux_apply_rope_2d(tk, ct, st, txt, H, D)
    r.ref_flux_apply_rope_2d(iq, ci, si, img, H, D)
    r.ref_flux_apply_rope_2d(ik, ci, si, img, H, D)
    g["flux_q_prologue"] = np.concatenate([tq, iq])
    g["flux_k_prologue"] = np.concatenate([tk, ik])
    io = np.zeros_like(iq); to = np.zeros_like(tq)
    assert r.ref_flux_joint_attention(io, to, iq, ik, iv, tq, tk, tv, img, txt, H, D) == 0
    g["flux_joint_out"] = np.concatenate([to, io])
    cat = lambda a, b: np.ascontiguousarray(np.concatenate([a, b]))
    so = np.zeros((txt + img, H * D), np.float32)
    assert r.ref_flux_mha(so, cat(tq, iq), cat(tk, ik), cat(tv, iv), txt + img, H, D) == 0
    g["flux_single_out"] = so

    # --- FLUX.3: joint_rope, prologue, chunked attention --------------------
    txt, ih, iw = 16, 4, 4
    rh = np.array([4, 2], np.int32); rw = np.array([4, 6], np.int32)
    total = txt + ih * iw + int((rh * rw).sum())
    c3 = np.zeros((total, D // 2), np.float32); s3 = np.zeros_like(c3)
    assert r.ref_f3_joint_rope(c3, s3, txt, ih, iw, rh, rw, 2, H, D, 10000.0) == total
    g["f3_rope_cos"], g["f3_rope_sin"] = c3, s3
    q3, k3, v3 = (ref_randn(r, 2000 + i, total, H * D) for i in range(3))
    r.ref_f3_head_rms_norm(q3, w_q, total, H, D, 1e-6)
    r.ref_f3_head_rms_norm(k3, w_k, total, H, D, 1e-6)
    r.ref_f3_apply_rope(q3, c3, s3, total, H, D)
    r.ref_f3_apply_rope(k3, c3, s3, total, H, D)
    g["f3_q_prologue"], g["f3_k_prologue"] = q3, k3
    o3 = np.zeros_like(q3)
    assert r.ref_f3_attention(o3, q3, k3, v3, total, H, D) == 0
    g["f3_out"] = o3

    # --- Z-Image: positions, prologue, masked attention ---------------------
    ht, wt, cap = 5, 6, 20                      # 30 image tokens -> 32, 20 caption -> 32
    o = ol.oracle()
    pos = np.zeros((64, 3), np.int32); mask = np.zeros(64, np.int32)
    seq = o.orc_zi_positions(pos.reshape(-1), mask, ht, wt, cap)
    assert seq == 64
    g["zi_pos"], g["zi_mask"] = pos, mask
    xz = ref_randn(r, 3000, seq, H * D)
    qz = xz.copy()
    ones = np.ones(D, np.float32)
    r.ref_zi_qk_norm(qz, ones, seq, H, D, 1e-5)
    r.ref_zi_apply_rope(qz, pos.reshape(-1), seq, H, D)
    g["zi_q_prologue"] = qz
    oz = np.zeros_like(xz)
    assert r.ref_zi_attention_identity(oz, xz, pos.reshape(-1), mask, seq, H, D) == 0
    g["zi_masked_out"] = oz
    oz2 = np.zeros_like(xz)
    assert r.ref_zi_attention_identity(oz2, xz, pos.reshape(-1), None, seq, H, D) == 0
    g["zi_unmasked_out"] = oz2

    path = os.path.join(HERE, "reference_cpu.npz")
    np.savez_compressed(path, **g)
    print("wrote", path, "%.1f KB" % (os.path.getsize(path) / 1024), "with", len(g), "arrays")


if __name__ == "__main__":
    main()
