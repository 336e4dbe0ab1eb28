#!/usr/bin/env python3
"""Generate tests/golden/reference_block.npz from the reference's own CPU code.

Run where the reference sources are present:

    make -C oracle ref && python tests/golden/make_block_golden.py

Records what the reference's single_block_forward and double_block_forward
(iris_transformer_flux.c:3341-3477, :2133-2327) and its FLUX.3 block_forward
(iris_transformer_flux3.c:371-417) and its Z-Image zi_block_forward
(iris_transformer_zimage.c:801-880), compiled unmodified into
oracle/_ref/libiris_ref_generic.so, make of the seeded inputs of
tests/block_cases.py. Inputs are not stored: block_cases regenerates them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import block_cases as bc  # noqa: E402
import oracle_lib as ol  # noqa: E402


ROW_STEP = {bc.SMALL["name"]: 1, bc.MID["name"]: 4}


def reference_block(r, case, inp):
    """x after the block by the reference's CPU code (its own RoPE tables)."""
    H, txt, (ih, iw) = case["heads"], case["txt"], case["img"]
    img = ih * iw
    ct = np.zeros((txt, bc.D), np.float32)
    st = np.zeros_like(ct)
    ci = np.zeros((img, bc.D), np.float32)
    si = np.zeros_like(ci)
    r.ref_flux_rope_text(ct, st, txt, 32, 2000.0)
    r.ref_flux_rope_2d(ci, si, ih, iw, 32, 2000.0)
    x = inp["x"].copy()
    rc = r.ref_flux_single_block(x, ol.from_bf16(inp["w_in"]), ol.from_bf16(inp["w_out"]), inp["norm_q"],
                                 inp["norm_k"], inp["t_emb"], inp["adaln"], ci, si, ct, st, inp["seq"], txt, H,
                                 bc.D, case["mlp"])
    assert rc == 0
    return x


def reference_double_block(r, case, inp):
    """x after a double block by the reference's CPU code: separate Q / K / V
    and gate / up matrices (the slices of the fused device weights), its own
    RoPE tables, text and image hidden states as separate arrays."""
    import ctypes as C
    H, txt, (ih, iw), dim, mlp = case["heads"], case["txt"], case["img"], inp["dim"], inp["mlp"]
    img = ih * iw
    ct = np.zeros((txt, bc.D), np.float32)
    st = np.zeros_like(ct)
    ci = np.zeros((img, bc.D), np.float32)
    si = np.zeros_like(ci)
    r.ref_flux_rope_text(ct, st, txt, 32, 2000.0)
    r.ref_flux_rope_2d(ci, si, ih, iw, 32, 2000.0)
    keep, ptrs = [], []
    for s in (inp["img"], inp["txt"]):
        qkv, ff_in = ol.from_bf16(s["qkv"]), ol.from_bf16(s["ff_in"])
        mats = [qkv[:dim], qkv[dim:2 * dim], qkv[2 * dim:], ol.from_bf16(s["proj"]), ff_in[:mlp], ff_in[mlp:],
                ol.from_bf16(s["ff_out"]), s["norm_q"], s["norm_k"]]
        mats = [np.ascontiguousarray(m, np.float32) for m in mats]
        keep.append(mats)
        ptrs.append((C.c_void_p * 9)(*[m.ctypes.data for m in mats]))
    xt, xi = inp["x"][:txt].copy(), inp["x"][txt:].copy()
    rc = r.ref_flux_double_block(xi, xt, ptrs[0], ptrs[1], inp["img"]["mod"], inp["txt"]["mod"], ci, si, ct, st,
                                 img, txt, H, bc.D, mlp)
    assert rc == 0
    return np.concatenate([xt, xi])


def reference_f3_block(r, case, inp):
    """x after a FLUX.3 block by the reference's CPU code: block_forward with
    the separate matrices that the fused device weights are made of."""
    import ctypes as C
    dim, mlp = inp["dim"], inp["mlp"]
    w_in, w_out = inp["w_in"], inp["w_out"]
    mats = [w_in[:dim], w_in[dim:2 * dim], w_in[2 * dim:3 * dim], w_out[:, :dim], w_in[3 * dim:], w_out[:, dim:]]
    mats = [np.ascontiguousarray(m) for m in mats]
    ptrs = (C.c_void_p * 6)(*[m.ctypes.data for m in mats])
    n = len(inp["seg_mod"])
    mods = (C.c_void_p * n)(*[m.ctypes.data for m in inp["seg_mod"]])
    x = inp["x"].copy()
    rc = r.ref_f3_block(x, ptrs, inp["norm_q"], inp["norm_k"], inp["seg_start"], inp["seg_len"], mods, n, inp["cos"],
                        inp["sin"], inp["seq"], inp["heads"], bc.D, mlp, case["eps"])
    assert rc == 0
    return x


def reference_zi_block(r, case, inp):
    """x after a Z-Image block by the reference's CPU code (zi_block_forward
    with the separate fp32 matrices the fused device weights are made of, its
    own RoPE tables from the position ids, the padding mask)."""
    import ctypes as C
    dim, ff, w = inp["dim"], inp["ff"], inp["w"]
    qkv, ff_in = ol.from_bf16(w["qkv"]), ol.from_bf16(w["ff_in"])
    mats = [qkv[:dim], qkv[dim:2 * dim], qkv[2 * dim:], ol.from_bf16(w["proj"]), ff_in[:ff], ff_in[ff:],
            ol.from_bf16(w["ff_out"]), w["attn_norm1"], w["attn_norm2"], w["ffn_norm1"], w["ffn_norm2"]]
    mats = [np.ascontiguousarray(m, np.float32) for m in mats]
    ptrs = (C.c_void_p * 11)(*[m.ctypes.data for m in mats])
    x = inp["x"].copy()
    rc = r.ref_zi_block(x, ptrs, w["norm_q"], w["norm_k"], inp["mod"], np.ascontiguousarray(inp["pos"].reshape(-1)),
                        inp["mask"], inp["seq"], inp["heads"], bc.D, ff)
    assert rc == 0
    return x


def main():
    r = ol.ref("generic")
    if r is None:
        sys.exit("oracle/_ref/libiris_ref_generic.so is missing: run `make -C oracle ref` first")
    out = {}
    for case in (bc.SMALL, bc.MID):
        inp = bc.block_inputs(case)
        # every row of the small case, every fourth of the other: the file stays small
        out[case["name"]] = reference_block(r, case, inp)[::ROW_STEP[case["name"]]]
        out[case["name"] + "/x_sum"] = np.float64(inp["x"].astype(np.float64).sum())
    for case in (bc.SMALL,):
        inp = bc.double_inputs(case)
        out["double/" + case["name"]] = reference_double_block(r, case, inp)
    for case in (bc.F3_SMALL,):
        inp = bc.f3_inputs(case)
        out["f3/" + case["name"]] = reference_f3_block(r, case, inp)[::2]          # every second row
    for case in (bc.ZI_SMALL,):
        inp = bc.zi_inputs(case)
        out["zi/" + case["name"]] = reference_zi_block(r, case, inp)[::2]          # every second row
    path = os.path.join(HERE, "reference_block.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
