"""Workloads of the joint-attention path and the GPU-vs-oracle comparison.

A case describes one transformer block's attention input the way the
reference produces it: token order, seeded N(0,1) Q/K/V rounded once to bf16,
unit norm weights, RoPE tables of the model family. ``run_case`` pushes it
through the C-ABI (prologue + attention on the strided views of a fused
[seq, 3*H*128] buffer, as the reference lays them out) and checks the result
against the CPU oracle on the same rounded inputs.

Synthetic stand-ins: the reference measures on no public dataset, so seeded
normal tensors with the models' shapes replace real activations.
"""
import ctypes as C

import numpy as np

import oracle_lib as ol

D = 128

# BASELINE configs (heads, token counts) and small versions of each family.
FLUX_CFG1 = dict(name="klein4b-256", family="flux2", heads=24, txt=512, img=(16, 16), refs=[], eps=1e-6)
FLUX_CFG2 = dict(name="klein4b-1024", family="flux2", heads=24, txt=512, img=(64, 64), refs=[], eps=1e-6)
FLUX_CFG3 = dict(name="klein9b-cfg", family="flux2", heads=32, txt=512, img=(64, 64), refs=[], eps=1e-6, batch=2)
ZIMAGE_CFG4 = dict(name="zimage-turbo", family="zimage", heads=30, txt=512, img=(64, 64), refs=[], eps=1e-5)
FLUX3_CFG5 = dict(name="flux3-multiref", family="flux3", heads=24, txt=512, img=(64, 64),
                  refs=[(64, 64)] * 3, eps=1e-6)

FLUX_SMALL = dict(name="flux2-small", family="flux2", heads=3, txt=40, img=(9, 11), refs=[], eps=1e-6)
FLUX_REF_SMALL = dict(name="flux2-ref-small", family="flux2", heads=2, txt=24, img=(8, 8), refs=[(8, 6)], eps=1e-6)
FLUX3_SMALL = dict(name="flux3-small", family="flux3", heads=2, txt=33, img=(10, 10), refs=[(6, 6), (5, 7)], eps=1e-6)
ZIMAGE_SMALL = dict(name="zimage-small-padded", family="zimage", heads=3, txt=50, img=(9, 13), refs=[], eps=1e-5)


def seq_len(case):
    n = case["txt"] + case["img"][0] * case["img"][1] + sum(h * w for h, w in case["refs"])
    if case["family"] == "zimage":
        ip = (case["img"][0] * case["img"][1] + 31) // 32 * 32
        cp = (case["txt"] + 31) // 32 * 32
        n = ip + cp
    return n


def rope_tables(case):
    """(cos, sin) [seq, 64] fp32 and the key mask (or None), in token order."""
    o = ol.oracle()
    fam, txt, (ih, iw) = case["family"], case["txt"], case["img"]
    seq = seq_len(case)
    cos = np.zeros((seq, 64), np.float32)
    sin = np.zeros_like(cos)
    mask = None
    if fam == "flux2":               # [TEXT, IMAGE, REFS], theta 2000, refs at T = 10 (i + 1)
        o.orc_flux_rope_text(cos[:txt], sin[:txt], txt, 32, 2000.0)
        off = txt
        for i, (h, w) in enumerate([(ih, iw)] + list(case["refs"])):
            o.orc_flux_rope_image(cos[off:off + h * w], sin[off:off + h * w], h, w, 32, 2000.0, 10 * i)
            off += h * w
    elif fam == "flux3":             # [TEXT, IMAGE, REFS], theta 10000, refs at l = -(i + 1)
        rh = np.array([h for h, _ in case["refs"]] or [0], np.int32)
        rw = np.array([w for _, w in case["refs"]] or [0], np.int32)
        n = o.orc_f3_joint_rope(cos, sin, txt, ih, iw, rh, rw, len(case["refs"]), D, 10000.0)
        assert n == seq
    else:                            # Z-Image [IMAGE | CAPTION], both padded to 32
        pos = np.zeros((seq, 3), np.int32)
        m = np.zeros(seq, np.int32)
        assert o.orc_zi_positions(pos.reshape(-1), m, ih, iw, txt) == seq
        o.orc_zi_rope(cos, sin, pos.reshape(-1), seq, 256.0)
        if not m.all():
            mask = m
    return cos, sin, mask


def qkv_inputs(case, b=0):
    """Seeded fp32 Q, K, V [seq, H*128]: image rows from seed 42 (shared by the
    cond / uncond batch entries), text rows from seed 1000 + b, reference
    image i from seed 2000 + i."""
    hd = case["heads"] * D
    seq, txt = seq_len(case), case["txt"]
    nimg = case["img"][0] * case["img"][1]
    q, k, v = (np.zeros((seq, hd), np.float32) for _ in range(3))

    def fill(rows, seed):
        block = ol.randn(seed, 3, rows.stop - rows.start, hd)
        q[rows], k[rows], v[rows] = block[0], block[1], block[2]

    if case["family"] == "zimage":
        ip = (nimg + 31) // 32 * 32
        fill(slice(0, nimg), 42)
        fill(slice(ip, ip + txt), 1000 + b)
    else:
        fill(slice(0, txt), 1000 + b)
        fill(slice(txt, txt + nimg), 42)
        off = txt + nimg
        for i, (h, w) in enumerate(case["refs"]):
            fill(slice(off, off + h * w), 2000 + i)
            off += h * w
    return q, k, v


def sample_rows(seq, n=96, seed=5):
    if seq <= 1024:
        return None
    rng = np.random.default_rng(seed)
    fixed = [0, 1, 127, 128, 255, 256, 511, 512, seq - 129, seq - 128, seq - 2, seq - 1]
    rows = np.unique(np.concatenate([np.array(fixed), rng.integers(0, seq, n)]))
    return rows.astype(np.int32)


def oracle_case(case, b=0, rows="auto"):
    """CPU result on the bf16-rounded inputs: prologue in fp32, attention on
    the sampled rows. Returns (out, q_pro, k_pro, rows)."""
    o = ol.oracle()
    H = case["heads"]
    q, k, v = qkv_inputs(case, b)
    for x in (q, k, v):
        o.orc_round_bf16(x.reshape(-1), x.size)
    cos, sin, mask = rope_tables(case)
    w = np.ones(D, np.float32)
    seq = q.shape[0]
    o.orc_head_norm_rope_f32(q.ctypes.data, H * D, w, cos, sin, seq, H, D, case["eps"], 0)
    o.orc_head_norm_rope_f32(k.ctypes.data, H * D, w, cos, sin, seq, H, D, case["eps"], 0)
    if rows == "auto":
        rows = sample_rows(seq)
    out = ol.dev_attention(q, k, v, H, key_mask=mask, rows=rows)
    return out, q, k, rows


class DeviceCase:
    """Device buffers of one case laid out as the reference's fused QKV
    activation: qkv [seq, 3*H*128] bf16 (ldi = 3*H*128), out [seq, H*128]."""

    def __init__(self, lib, case, b=0):
        self.lib, self.case = lib, case
        H = case["heads"]
        self.H, self.hd, self.seq = H, H * D, seq_len(case)
        q, k, v = qkv_inputs(case, b)
        fused = np.concatenate([q, k, v], axis=1)
        self.host_qkv = ol.to_bf16(fused)
        cos, sin, mask = rope_tables(case)
        self.cos_h, self.sin_h, self.mask_h = cos, sin, mask
        self.qkv = lib.to_device(self.host_qkv)
        self.cos = lib.to_device(cos)
        self.sin = lib.to_device(sin)
        self.w = lib.to_device(np.ones(D, np.float32))
        self.mask = lib.to_device(mask) if mask is not None else None
        self.out = lib.alloc(self.seq * self.hd * 2)
        self.ldi = 3 * self.hd

    def ptr(self, which):
        return C.c_void_p(self.qkv + {"q": 0, "k": 1, "v": 2}[which] * self.hd * 2)

    def reset(self):
        self.lib.iris_dev_upload(self.qkv, self.host_qkv.ctypes.data, self.host_qkv.nbytes)

    def prologue(self, fused=True):
        lib, c = self.lib, self.case
        if fused:
            rc = lib.iris_b200_qk_norm_rope(self.ptr("q"), self.ptr("k"), self.ldi, self.w, self.w,
                                            self.cos, self.sin, self.seq, self.H, D, c["eps"], 0)
            assert rc == 0, rc
        else:
            for which in ("q", "k"):
                lib.iris_dev_head_norm_rope(self.ptr(which), self.ldi, self.w, self.cos, self.sin,
                                            self.seq, self.H, D, c["eps"], 0)

    def attention(self, kernel=0):
        rc = self.lib.iris_b200_attention_ex(self.out, self.hd, self.ptr("q"), self.ptr("k"), self.ptr("v"),
                                             self.ldi, self.seq, self.seq, self.H, self.H, D,
                                             1.0 / np.sqrt(D), 0, self.mask, kernel)
        assert rc == 0, rc

    def read_out(self):
        return ol.from_bf16(self.lib.to_host(self.out, (self.seq, self.hd), np.uint16))

    def read_qkv(self):
        return self.lib.to_host(self.qkv, (self.seq, 3 * self.hd), np.uint16)

    def free(self):
        for p in (self.qkv, self.cos, self.sin, self.w, self.mask, self.out):
            if p:
                self.lib.iris_dev_free(p)


def run_case(lib, case, kernel=0, b=0, fused_prologue=True, rows="auto"):
    """Prologue + attention on the GPU vs the oracle. Returns the metrics the
    parity gate is stated in: per-head max abs error and cosine."""
    dc = DeviceCase(lib, case, b)
    try:
        dc.prologue(fused_prologue)
        dc.attention(kernel)
        got = dc.read_out()
        qkv = dc.read_qkv()
        lib.check()
    finally:
        dc.free()
    want, q_pro, k_pro, rows = oracle_case(case, b, rows)
    H = case["heads"]
    mx, cs = ol.compare_heads(got, want, H, D, rows)
    # prologue alone: bf16 result vs fp32 oracle, relative to bf16 resolution
    qg = ol.from_bf16(qkv[:, :H * D])
    kg = ol.from_bf16(qkv[:, H * D:2 * H * D])
    pro_err = max(np.abs(qg - q_pro).max(), np.abs(kg - k_pro).max())
    return dict(max_abs=float(mx.max()), min_cos=float(cs.min()), per_head_max=mx, per_head_cos=cs,
                prologue_max_abs=float(pro_err), rows=rows, out=got, want=want)


def write_block_input(path, case, b=0):
    """Input file of the C host program (iris.c_b200/examples/block_attention.c)."""
    H = case["heads"]
    q, k, v = qkv_inputs(case, b)
    cos, sin, mask = rope_tables(case)
    assert mask is None
    with open(path, "wb") as f:
        f.write(np.array([seq_len(case), H], np.int32).tobytes())
        f.write(np.array([case["eps"]], np.float32).tobytes())
        f.write(ol.to_bf16(np.concatenate([q, k, v], axis=1)).tobytes())
        f.write(cos.tobytes())
        f.write(sin.tobytes())
        f.write(np.ones(D, np.float32).tobytes())
        f.write(np.ones(D, np.float32).tobytes())
