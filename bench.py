#!/usr/bin/env python3
"""Benchmark of the joint-attention hot path (prologue + attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload NAME] [--mode MODE]

One step = one pass of the hot path over one transformer block's input: the
Q/K prologue (per-head RMSNorm + RoPE, in place on the fused QKV activation)
followed by the joint attention, through the C-ABI of libiris_b200.so.
Metric: attention TFLOP/s, 4*B*H*S^2*128 FLOP per step (QK^T and PV; softmax,
scaling and prologue not counted), aggregate over all GPUs of the job.

N = 1 runs the Klein-4B 1024^2 block (4608 tokens, 24 heads, bf16). N > 1
runs the FLUX.3 multi-reference block (16 896 tokens, 24 heads) with ring
sequence parallelism: every GPU keeps its token rows, the K/V rows travel
peer to peer while one attention launch per GPU consumes them. The same
line carries, as extra keys, that workload on one GPU measured in the same
run (`speedup_vs_1gpu`), its head-parallel decomposition, and the
independent-shard runs of the Klein-9B CFG block (cond/uncond x heads) and of
the Z-Image block (30 heads, uneven split).

Data is synthetic: seeded N(0,1) Q/K/V in bf16, unit norm weights and the
RoPE tables of the model family; the reference publishes no dataset for this
path. Inputs rotate through several buffer sets larger than L2 in total.

Parity inside the run: the CPU leg (the reference's own CPU code) consumes
the very tensors the GPU arm uploaded (the bf16 values widened to fp32) and
the line reports the worst per-head max-abs error and cosine between the two
results (`parity`).

--impl reference times the reference's own CPU implementation of the same
step (oracle/_ref, built from the reference sources; else the CPU port in
oracle/) on the host cores, on a bounded sample of the workload.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
D = 128

WORKLOADS = {
    # name: family, heads, text tokens, image grid, reference grids, batch, eps
    "klein4b-256": dict(family="flux2", heads=24, txt=512, img=(16, 16), refs=[], batch=1, eps=1e-6),
    "klein4b-1024": dict(family="flux2", heads=24, txt=512, img=(64, 64), refs=[], batch=1, eps=1e-6),
    "klein9b-cfg": dict(family="flux2", heads=32, txt=512, img=(64, 64), refs=[], batch=2, eps=1e-6),
    "zimage-turbo": dict(family="zimage", heads=30, txt=512, img=(64, 64), refs=[], batch=1, eps=1e-5),
    # 4224 tokens: the per-rank chunk of flux3-multiref on 8 GPUs, as a 2-rank ring probe
    "flux3-short": dict(family="flux3", heads=24, txt=512, img=(58, 64), refs=[], batch=1, eps=1e-6),
    "flux3-multiref": dict(family="flux3", heads=24, txt=512, img=(64, 64), refs=[(64, 64)] * 3, batch=1, eps=1e-6),
}


# DRAM bytes (read + written) of one attention launch as counted by an ncu capture of this workload
# (dram__bytes_read.sum + dram__bytes_write.sum); not measured by this script. The algorithmic
# figure for comparison is Q + K + V + O = 113.2 MB.
NCU_DRAM_BYTES_PER_LAUNCH = {"klein4b-1024": 90.3e6}

METRIC = "joint-attn TFLOP/s per GPU & % bf16 peak at 1/2/4/8 B200 vs host-CPU ref"
STEP_WORDS = "qk_norm + rope + attention"


def seq_len(w):
    return w["txt"] + w["img"][0] * w["img"][1] + sum(h * x for h, x in w["refs"])


def attn_flops(batch, heads, sq, sk):
    return 4.0 * batch * heads * sq * sk * D


# ---------------------------------------------------------------------------
# synthetic inputs (no oracle code here: plain numpy / torch)
# ---------------------------------------------------------------------------

def axis_angles(pos, n, axis_dim, theta):
    omega = 1.0 / (theta ** (np.arange(0, 2 * n, 2, dtype=np.float64) / axis_dim))
    return np.asarray(pos, np.float64)[:, None] * omega[None, :]


def rope_tables(w):
    """cos / sin [seq, 64] fp32 in the token order of the family."""
    txt, (ih, iw) = w["txt"], w["img"]
    grids = [(ih, iw)] + list(w["refs"])
    rows = []
    if w["family"] == "flux2":        # (T, H, W, L) x 16 pairs, theta 2000, refs at T = 10 i
        z = np.zeros(txt)
        rows.append(np.concatenate([axis_angles(z, 16, 32, 2000.0)] * 3 +
                                   [axis_angles(np.arange(txt), 16, 32, 2000.0)], 1))
        for i, (h, x) in enumerate(grids):
            yy, xx = np.divmod(np.arange(h * x), x)
            rows.append(np.concatenate([axis_angles(np.full(h * x, 10.0 * i), 16, 32, 2000.0),
                                        axis_angles(yy, 16, 32, 2000.0), axis_angles(xx, 16, 32, 2000.0),
                                        axis_angles(np.zeros(h * x), 16, 32, 2000.0)], 1))
    elif w["family"] == "flux3":      # theta 10000, half-step grid, refs at l = -(i + 1)
        z = np.zeros(txt)
        rows.append(np.concatenate([axis_angles(z, 16, 32, 1e4)] * 3 + [axis_angles(np.arange(txt), 16, 32, 1e4)], 1))
        for i, (h, x) in enumerate(grids):
            yy, xx = np.divmod(np.arange(h * x), x)
            rows.append(np.concatenate([axis_angles(np.zeros(h * x), 16, 32, 1e4), axis_angles(0.5 * yy, 16, 32, 1e4),
                                        axis_angles(0.5 * xx, 16, 32, 1e4),
                                        axis_angles(np.full(h * x, -float(i)), 16, 32, 1e4)], 1))
    else:                             # Z-Image [IMAGE | CAPTION], axes 32/48/48, theta 256
        n = ih * iw
        yy, xx = np.divmod(np.arange(n), iw)
        rows.append(np.concatenate([axis_angles(np.full(n, txt + 1), 16, 32, 256.0), axis_angles(yy, 24, 48, 256.0),
                                    axis_angles(xx, 24, 48, 256.0)], 1))
        rows.append(np.concatenate([axis_angles(1 + np.arange(txt), 16, 32, 256.0),
                                    axis_angles(np.zeros(txt), 24, 48, 256.0),
                                    axis_angles(np.zeros(txt), 24, 48, 256.0)], 1))
    ang = np.concatenate(rows, 0)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def make_qkv(seq, width, seed):
    """Pinned bf16 [seq, 3*width] N(0,1) (torch is used for the generator and
    the page-locked allocation only)."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    buf = torch.empty((seq, 3 * width), dtype=torch.bfloat16)
    if torch.cuda.is_available():
        buf = buf.pin_memory()
    step = 512
    for r0 in range(0, seq, step):
        r1 = min(seq, r0 + step)
        buf[r0:r1] = torch.randn((r1 - r0, 3 * width), generator=gen).to(torch.bfloat16)
    return buf


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for t, l in self.lines if t0 - 0.05 <= t <= t1 + 0.15]
        if not rows:
            rows = [l.split(", ") for _, l in self.lines[-3:]]
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# the B200 arm
# ---------------------------------------------------------------------------

def load_lib():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    return ge.load_package().load()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p.get("bf16_tflops", 1632.7), p.get("bf16_tflops_sustained", 1365.4), p.get("hbm_gbs", 6551.0), "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


class Job:
    """Process-wide state of one bench run: the library, this rank, the
    process group."""

    def __init__(self):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
        self.lib = load_lib()
        self.lib.init(self.local)
        self.ring_ready = False

    def barrier(self, group_all=True):
        if self.dist and group_all:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if not self.dist:
            return list(values)
        t = self.torch.tensor(list(values), device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def ring_init(self, parts=0, groups=1):
        """One ring per head group: the ranks [g * R, (g + 1) * R) with R =
        world / groups form ring g; its first rank makes the ring's id."""
        if self.ring_ready:
            return
        torch, lib = self.torch, self.lib
        assert self.world % groups == 0
        size = self.world // groups
        leader = self.rank - self.rank % size
        assert lib.iris_b200_ring_configure(0, parts) == 0
        mine = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if self.rank == leader:
            buf = C.create_string_buffer(128)
            assert lib.iris_b200_ring_unique_id(buf) == 0
            mine = torch.tensor(list(buf.raw), dtype=torch.uint8, device="cuda")
        ids = [mine]
        if self.dist:
            ids = [torch.zeros_like(mine) for _ in range(self.world)]
            self.dist.all_gather(ids, mine)
        assert lib.iris_b200_ring_init(self.rank - leader, size, bytes(ids[leader].cpu().tolist())) == 0
        self.ring_ready = True

    def ring_destroy(self):
        if self.ring_ready:
            self.lib.iris_b200_ring_destroy()
            self.ring_ready = False


def plan_of(job, w, mode, groups=1):
    """What this rank holds and computes. mode: 'single' (everything on this
    rank), 'shard' (batch entries on disjoint GPU groups, heads of an entry
    split over its group: independent shards, nothing exchanged) or 'ring'
    (this rank's block of token rows; with `groups` > 1 the heads are split
    over that many independent rings of world / groups ranks each)."""
    lib, rank, world = job.lib, job.rank, job.world
    S_full, H = seq_len(w), w["heads"]
    p = dict(mode=mode, S_full=S_full, S=S_full, row0=0, rows_of=None, entries=list(range(w["batch"])), h0=0, nh=H)
    a, b, c, d = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    if mode == "shard":
        assert lib.iris_b200_cfg_shard(w["batch"], H, world, rank, C.byref(a), C.byref(b), C.byref(c), C.byref(d)) == 0
        p["entries"] = list(range(a.value, w["batch"], b.value)) if d.value > 0 else []
        p["h0"], p["nh"] = c.value, d.value
    elif mode == "ring":
        assert w["batch"] == 1 and world % groups == 0
        size = world // groups
        grp, rr = rank // size, rank % size
        rows_of = np.zeros(size, np.int32)
        for r in range(size):
            lib.iris_b200_seq_shard(S_full, size, r, C.byref(a), C.byref(b))
            rows_of[r] = b.value
            if r == rr:
                p["row0"] = a.value
        p["rows_of"], p["S"], p["groups"] = rows_of, int(rows_of[rr]), groups
        if groups > 1:
            assert lib.iris_b200_head_shard(H, groups, grp, C.byref(c), C.byref(d)) == 0
            p["h0"], p["nh"] = c.value, d.value
    return p


class Buffers:
    """Device buffer sets of one plan: each set holds, per batch entry of this
    rank, the fused QKV slice [S, 3 * width] and the output [S, width]; enough
    sets to exceed L2 (126 MB) several times. The host copies are the pinned
    tensors every set was uploaded from."""

    def __init__(self, job, w, plan, seed_base=None):
        lib = job.lib
        self.job, self.w, self.plan = job, w, plan
        S, nh = plan["S"], plan["nh"]
        self.width = nh * D
        cos, sin = rope_tables(w)
        self.cos = np.ascontiguousarray(cos[plan["row0"]:plan["row0"] + S])
        self.sin = np.ascontiguousarray(sin[plan["row0"]:plan["row0"] + S])
        self.d_cos, self.d_sin = lib.to_device(self.cos), lib.to_device(self.sin)
        self.d_w = lib.to_device(np.ones(D, np.float32))
        entries = plan["entries"] if nh > 0 else []
        self.per_set = len(entries) * S * self.width * 8
        self.nsets = max(2, min(8, int(np.ceil(512e6 / max(self.per_set, 1))))) if entries else 0
        seed_base = 1000 * job.rank if seed_base is None else seed_base
        self.host_qkv = [make_qkv(S, self.width, seed_base + e) for e in entries]
        self.sets = []
        for _ in range(self.nsets):
            bufs = []
            for hq in self.host_qkv:
                dq = lib.alloc(hq.numel() * 2)
                lib.iris_dev_upload(dq, hq.data_ptr(), hq.numel() * 2)
                bufs.append((dq, lib.alloc(S * self.width * 2)))
            self.sets.append(bufs)
        lib.check()

    def free(self):
        lib = self.job.lib
        for bufs in self.sets:
            for dq, dout in bufs:
                lib.iris_dev_free(dq)
                lib.iris_dev_free(dout)
        for p in (self.d_cos, self.d_sin, self.d_w):
            lib.iris_dev_free(p)
        self.sets = []


def run_step(job, w, plan, B, bufs, cs=None, mark=None):
    """One step on one buffer set: per batch entry the Q/K prologue, then the
    attention (plain, or the ring call)."""
    lib = job.lib
    S, nh, width = plan["S"], plan["nh"], B.width
    scale = 1.0 / np.sqrt(D)
    d_cos, d_sin = cs if cs else (B.d_cos, B.d_sin)
    for dq, dout in bufs:
        q, k, v = dq, dq + width * 2, dq + 2 * width * 2
        if mark is not None:
            lib.iris_b200_mark(mark + 2)
        lib.iris_b200_qk_norm_rope(q, k, 3 * width, B.d_w, B.d_w, d_cos, d_sin, S, nh, D, w["eps"], 0)
        if mark is not None:
            lib.iris_b200_mark(mark)
        if plan["mode"] == "ring":
            rc = lib.iris_b200_ring_attention(dout, width, q, k, v, 3 * width, plan["rows_of"].ctypes.data, nh, scale)
            assert rc == 0, rc
        else:
            lib.iris_dev_attention(dout, width, q, k, v, 3 * width, S, S, nh, nh, D, scale, 0, None)
        if mark is not None:
            lib.iris_b200_mark(mark + 1)


def timed_steps(job, w, plan, B, steps, warmup, collective=True, marks=False):
    """W warm-up steps, then K steps between two marks on the library's
    stream, bracketed by a barrier + device synchronisation. Returns the time
    per step in ms (max over the ranks when `collective`), the launches
    enqueued and, with marks, the durations of the attention and prologue
    launches of every step."""
    lib = job.lib
    active = bool(B.sets)
    for i in range(warmup):
        if active:
            run_step(job, w, plan, B, B.sets[i % B.nsets])
    job.barrier(collective)
    launches0 = lib.iris_b200_launch_count()
    t0 = time.time()
    lib.iris_b200_mark(0)
    # Per-kernel marks on every fourth step of the timed region: an event record
    # between the prologue and the attention launch costs that step the overlap
    # of the two (programmatic stream serialisation), so the others run clean.
    marked = [i for i in range(2 if steps > 2 else 0, steps, 4)][:2500] if (marks and active and len(B.sets[0]) == 1) else []
    slot = {i: k for k, i in enumerate(marked)}
    for i in range(steps):
        if active:
            run_step(job, w, plan, B, B.sets[i % B.nsets], mark=2 + 3 * slot[i] if i in slot else None)
    lib.iris_b200_mark(1)
    t_enq = time.time()
    job.barrier(collective)
    t1 = time.time()
    ms = lib.iris_b200_mark_elapsed_ms(0, 1) / steps
    lib.check()
    if collective:
        ms = job.max_over_ranks([ms])[0]
    res = dict(ms=ms, launches=int(lib.iris_b200_launch_count() - launches0), wall=(t0, t1),
               enqueue_ms=(t_enq - t0) * 1e3 / steps)
    if marked:
        n = len(marked)
        res["attn_ms"] = [d for d in (lib.iris_b200_mark_elapsed_ms(2 + 3 * i, 3 + 3 * i) for i in range(n)) if d > 0]
        res["pro_ms"] = [d for d in (lib.iris_b200_mark_elapsed_ms(4 + 3 * i, 2 + 3 * i) for i in range(n)) if d > 0]
    return res


def e2e_steps(job, w, plan, B, steps):
    """End to end through the C-ABI with host buffers. Every step uploads its
    inputs (QKV slice and RoPE tables) from page-locked host memory, runs
    prologue + attention and downloads the result. `serial`: the reference's
    blocking iris_dev_upload / iris_dev_download around every step.
    `pipelined` (the reported value): iris_b200_upload_async /
    iris_b200_download_async on two copy streams of the library's making,
    ordered against the library's stream by events over three device buffer
    sets, so the upload of step i + 1 and the download of step i - 1 run under
    the kernels of step i. Returns ms per step (max over ranks) of both."""
    lib, torch = job.lib, job.torch
    S, width = plan["S"], B.width
    entries = B.host_qkv
    if not entries:
        r = job.max_over_ranks([0.0, 0.0])
        return r[0], r[1], 0, 0
    in_bytes, out_bytes = S * 3 * width * 2, S * width * 2
    cs_bytes = B.cos.nbytes
    nrep = max(1, min(steps, 10))
    host_out = lib.iris_b200_host_alloc(out_bytes)
    job.barrier()
    t0 = time.perf_counter()
    for i in range(nrep):
        bufs = B.sets[i % B.nsets]
        for (dq, dout), hq in zip(bufs, entries):
            lib.iris_dev_upload(dq, hq.data_ptr(), in_bytes)
        lib.iris_dev_upload(B.d_cos, B.cos.ctypes.data, cs_bytes)
        lib.iris_dev_upload(B.d_sin, B.sin.ctypes.data, cs_bytes)
        run_step(job, w, plan, B, bufs)
        for dq, dout in bufs:
            lib.iris_dev_download(host_out, dout, out_bytes)
    torch.cuda.synchronize()
    serial_ms = (time.perf_counter() - t0) * 1e3 / nrep

    nbuf, prep = 3, max(3, min(steps, 30))
    up, down = lib.iris_b200_stream_create(), lib.iris_b200_stream_create()
    pin_cos, pin_sin = lib.iris_b200_host_alloc(cs_bytes), lib.iris_b200_host_alloc(cs_bytes)
    C.memmove(pin_cos, B.cos.ctypes.data, cs_bytes)
    C.memmove(pin_sin, B.sin.ctypes.data, cs_bytes)
    dev = [[(lib.alloc(in_bytes), lib.alloc(out_bytes)) for _ in entries] for _ in range(nbuf)]
    dev_cs = [(lib.alloc(cs_bytes), lib.alloc(cs_bytes)) for _ in range(nbuf)]
    pin_out = [[lib.iris_b200_host_alloc(out_bytes) for _ in entries] for _ in range(nbuf)]
    ev_up = [lib.iris_b200_event_create() for _ in range(prep)]
    ev_comp = [lib.iris_b200_event_create() for _ in range(prep)]
    ev_down = [lib.iris_b200_event_create() for _ in range(prep)]
    job.barrier()
    t0 = time.perf_counter()
    for i in range(prep):
        b = i % nbuf
        if i >= nbuf:
            lib.iris_b200_stream_wait_event(up, ev_comp[i - nbuf])        # the last reader of this input set
        for (dq, _), hq in zip(dev[b], entries):
            lib.iris_b200_upload_async(dq, hq.data_ptr(), in_bytes, up)
        lib.iris_b200_upload_async(dev_cs[b][0], pin_cos, cs_bytes, up)
        lib.iris_b200_upload_async(dev_cs[b][1], pin_sin, cs_bytes, up)
        lib.iris_b200_event_record(ev_up[i], up)
        lib.iris_b200_stream_wait_event(None, ev_up[i])
        if i >= nbuf:
            lib.iris_b200_stream_wait_event(None, ev_down[i - nbuf])      # the last download of this output set
        run_step(job, w, plan, B, dev[b], cs=dev_cs[b])
        lib.iris_b200_event_record(ev_comp[i], None)
        lib.iris_b200_stream_wait_event(down, ev_comp[i])
        for (_, dout), po in zip(dev[b], pin_out[b]):
            lib.iris_b200_download_async(po, dout, out_bytes, down)
        lib.iris_b200_event_record(ev_down[i], down)
    lib.iris_b200_stream_sync(up)
    lib.iris_b200_stream_sync(down)
    lib.iris_b200_stream_sync(None)
    e_ms = (time.perf_counter() - t0) * 1e3 / prep
    lib.check()
    for ev in ev_up + ev_comp + ev_down:
        lib.iris_b200_event_destroy(ev)
    for st in (up, down):
        lib.iris_b200_stream_destroy(st)
    for row in dev:
        for dq, dout in row:
            lib.iris_dev_free(dq)
            lib.iris_dev_free(dout)
    for a, b in dev_cs:
        lib.iris_dev_free(a)
        lib.iris_dev_free(b)
    for p in [host_out, pin_cos, pin_sin] + [x for row in pin_out for x in row]:
        lib.iris_b200_host_free(p)
    e_ms, serial_ms = job.max_over_ranks([e_ms, serial_ms])
    return e_ms, serial_ms, len(entries) * (in_bytes + 2 * cs_bytes), len(entries) * out_bytes


def bf16_to_f32(t):
    """torch bf16 tensor -> numpy fp32 (exact widening)."""
    return t.float().numpy()


def head_errors(got, want, heads):
    """Worst per-head max-abs error and cosine between two fp32 [rows, heads * 128] results."""
    g = got.reshape(got.shape[0], heads, D).astype(np.float64)
    w = want.reshape(want.shape[0], heads, D).astype(np.float64)
    mx = np.abs(g - w).max(axis=(0, 2))
    cs = (g * w).sum(axis=(0, 2)) / np.sqrt((g * g).sum(axis=(0, 2)) * (w * w).sum(axis=(0, 2)) + 1e-300)
    return float(mx.max()), float(cs.min())


def gpu_result(job, w, plan, B):
    """One step on freshly uploaded inputs of buffer set 0; the output of
    batch entry 0 as fp32 [S, width]."""
    lib, torch = job.lib, job.torch
    if not B.sets:
        return None
    dq, dout = B.sets[0][0]
    hq = B.host_qkv[0]
    lib.iris_dev_upload(dq, hq.data_ptr(), hq.numel() * 2)
    run_step(job, w, plan, B, B.sets[0][:1])
    out = torch.empty((plan["S"], B.width), dtype=torch.bfloat16)
    lib.iris_dev_download(out.data_ptr(), dout, out.numel() * 2)
    lib.check()
    return out


def roofline_of(res, name, nh, S, S_full, pk):
    """Roofline objects of the two kernels of a step from the per-launch marks."""
    bf16_peak, bf16_sust, hbm_peak, src = pk
    roof = pro = None
    durs, pdurs = res.get("attn_ms") or [], res.get("pro_ms") or []
    if durs:
        kms = sum(durs) / len(durs)
        achieved = attn_flops(1, nh, S, S_full) / (kms * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": "k_attention_sm100", "achieved": round(achieved, 1),
                "peak": bf16_peak, "peak_source": src + " bf16 burst", "unit": "TFLOP/s",
                "frac": round(achieved / bf16_peak, 4), "frac_of_sustained": round(achieved / bf16_sust, 4),
                "kernel_ms": round(kms, 4), "kernel_ms_median": round(float(np.median(durs)), 4),
                "kernel_ms_min": round(min(durs), 4), "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(name),
                "traffic_source": "ncu capture of this workload (constant, not measured in this run)"
                if name in NCU_DRAM_BYTES_PER_LAUNCH else None}
    if pdurs:
        pms = sum(pdurs) / len(pdurs)
        pbytes = 4.0 * S * nh * D * 2 + 2.0 * S * 64 * 4     # Q and K read + written, cos + sin read
        pro = {"bound": "hbm", "kernel": "k_head_norm_rope_128_tok", "achieved": round(pbytes / pms / 1e6, 1),
               "peak": hbm_peak, "peak_source": src + " HBM copy", "unit": "GB/s",
               "frac": round(pbytes / pms / 1e6 / hbm_peak, 4), "kernel_ms": round(pms, 4),
               "kernel_ms_median": round(float(np.median(pdurs)), 4), "kernel_ms_min": round(min(pdurs), 4),
               "bytes": pbytes}
    return roof, pro


def projection_run(job, w, pk, reps=20):
    """The step before the path (rank 0, N = 1): the QKV projection of one
    block, [tokens, dim] x [3 dim, dim]^T, as the fused tcgen05 GEMM whose
    epilogue is the prologue, next to cuBLAS (torch.matmul) followed by the
    separate prologue kernel on the same device."""
    lib, torch = job.lib, job.torch
    S, H = seq_len(w), w["heads"]
    dim, out = H * D, 3 * H * D
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((S, dim), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    W = (torch.randn((out, dim), generator=gen, device="cuda", dtype=torch.float32) / dim ** 0.5).to(torch.bfloat16)
    ys = [torch.empty((S, out), device="cuda", dtype=torch.bfloat16) for _ in range(4)]      # 4 x 85 MB: beyond L2
    cos, sin = rope_tables(w)
    d_cos, d_sin, d_w = lib.to_device(cos), lib.to_device(sin), lib.to_device(np.ones(D, np.float32))
    torch.cuda.synchronize()

    def fused(i):
        rc = lib.iris_b200_linear_qk_norm_rope(ys[i % 4].data_ptr(), out, x.data_ptr(), W.data_ptr(), S, dim, out, H,
                                               d_w, d_w, d_cos, d_sin, w["eps"])
        assert rc == 0, rc

    def timed(fn):
        for i in range(3):
            fn(i)
        lib.iris_dev_sync()
        lib.iris_b200_mark(0)
        for i in range(reps):
            fn(i)
        lib.iris_b200_mark(1)
        return lib.iris_b200_mark_elapsed_ms(0, 1) / reps

    fused_ms = timed(fused)
    lib.check()
    # cuBLAS + separate prologue on the library's stream
    comp = torch.cuda.ExternalStream(int(lib.iris_b200_stream()))

    def blas(i):
        with torch.cuda.stream(comp):
            torch.matmul(x, W.t(), out=ys[i % 4])

    def blas_pro(i):
        blas(i)
        y = ys[i % 4].data_ptr()
        lib.iris_b200_qk_norm_rope(y, y + dim * 2, out, d_w, d_w, d_cos, d_sin, S, H, D, w["eps"], 0)

    blas_ms = timed(blas)
    both_ms = timed(blas_pro)
    lib.check()
    for p in (d_cos, d_sin, d_w):
        lib.iris_dev_free(p)
    flops = 2.0 * S * dim * out
    return {"shape": [S, dim, out], "kernel": "k_linear_sm100 (GEMM + RMSNorm + RoPE epilogue)",
            "ms": round(fused_ms, 4), "tflops": round(flops / fused_ms / 1e9, 1),
            "frac_of_bf16_peak": round(flops / fused_ms / 1e9 / pk[0], 4),
            "cublas_ms": round(blas_ms, 4), "cublas_tflops": round(flops / blas_ms / 1e9, 1),
            "cublas_plus_prologue_ms": round(both_ms, 4),
            "speedup_vs_cublas_plus_prologue": round(both_ms / fused_ms, 3)}


def block_run(job, w, pk, reps=10):
    """One whole single-stream block around the path (rank 0, N = 1): LayerNorm
    with modulation, the fused QKV+MLP projection with the prologue, attention,
    SwiGLU and the output projection with the gated residual - four launches
    through iris_b200_single_block - next to the reference's own CUDA backend
    issuing its eight calls (iris_transformer_flux.c:3828-3845) on the same
    device, where that build is present."""
    lib, torch = job.lib, job.torch
    S, H = seq_len(w), w["heads"]
    dim, mlp = H * D, 3 * H * D
    ldh, ldc = 3 * dim + 2 * mlp, dim + mlp
    gen = torch.Generator(device="cuda").manual_seed(9)

    def rnd(shape, scale=1.0, dtype=torch.float32):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * scale).to(dtype)

    x0 = rnd((S, dim))
    x = x0.clone()
    w_in, w_out = rnd((ldh, dim), dim ** -0.5, torch.bfloat16), rnd((dim, ldc), ldc ** -0.5, torch.bfloat16)
    nq, nk, mod = 1 + 0.1 * rnd((D,)), 1 + 0.1 * rnd((D,)), rnd((3 * dim,), 0.3)
    cos, sin = rope_tables(w)
    d_cos, d_sin = lib.to_device(cos), lib.to_device(sin)
    nbytes = lib.iris_b200_single_block_scratch_bytes(S, dim, mlp)
    scratch = lib.alloc(nbytes)
    torch.cuda.synchronize()

    def ours():
        rc = lib.iris_b200_single_block(x.data_ptr(), scratch, w_in.data_ptr(), w_out.data_ptr(), nq.data_ptr(),
                                        nk.data_ptr(), mod.data_ptr(), d_cos, d_sin, S, dim, H, mlp, None)
        assert rc == 0, rc

    for _ in range(3):
        ours()
    lib.iris_dev_sync()
    n0 = lib.iris_b200_launch_count()
    lib.iris_b200_mark(0)
    for _ in range(reps):
        ours()
    lib.iris_b200_mark(1)
    ms = lib.iris_b200_mark_elapsed_ms(0, 1) / reps
    launches = (lib.iris_b200_launch_count() - n0) // reps
    lib.check()
    # the same four launches one by one, a mark after each
    norm = scratch
    up256 = lambda b: (b + 255) & ~255
    qkv = scratch + up256(S * dim * 2)
    cat = qkv + up256(S * 3 * dim * 2)
    stages = ["layer_norm_mod", "qkv_mlp_projection+prologue+swiglu", "attention", "out_projection+residual"]
    acc = [0.0] * 4
    for r in range(reps):
        lib.iris_b200_mark(0)
        lib.iris_dev_layer_norm_mod(norm, x.data_ptr(), mod.data_ptr(), mod.data_ptr() + 4 * dim, S, dim, 1e-6)
        lib.iris_b200_mark(1)
        lib.iris_b200_linear_glu(qkv, 3 * dim, cat + 2 * dim, ldc, norm, w_in.data_ptr(), S, dim, H, mlp, nq.data_ptr(),
                                 nk.data_ptr(), d_cos, d_sin, 1e-6)
        lib.iris_b200_mark(2)
        lib.iris_dev_attention(cat, ldc, qkv, qkv + 2 * dim, qkv + 4 * dim, 3 * dim, S, S, H, H, D, 1.0 / np.sqrt(D), 0, None)
        lib.iris_b200_mark(3)
        lib.iris_b200_linear_residual(x.data_ptr(), dim, cat, ldc, w_out.data_ptr(), ldc, mod.data_ptr() + 8 * dim, S,
                                      ldc, dim)
        lib.iris_b200_mark(4)
        for i in range(4):
            acc[i] += lib.iris_b200_mark_elapsed_ms(i, i + 1)
    lib.check()
    flops = 2.0 * S * dim * ldh + 4.0 * S * S * dim + 2.0 * S * ldc * dim
    out = {"shape": {"tokens": S, "dim": dim, "heads": H, "mlp": mlp}, "launches_per_block": int(launches),
           "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
           "frac_of_bf16_sustained": round(flops / ms / 1e9 / pk[1], 4),
           "stage_ms": {n: round(a / reps, 4) for n, a in zip(stages, acc)}}
    # the reference's CUDA backend: eight calls per block, wall clock between its stream syncs
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    ref = ol.ref_cuda()
    if ref is not None and ref.iris_dev_init() == 1:
        proj = torch.empty((S, dim), device="cuda", dtype=torch.float32)
        r_h = torch.empty((S, ldh), device="cuda", dtype=torch.bfloat16)         # the reference's d->h
        h = r_h.data_ptr()
        xr = x0.clone()
        torch.cuda.synchronize()

        def theirs():
            ref.iris_dev_layer_norm_mod(norm, xr.data_ptr(), mod.data_ptr(), mod.data_ptr() + 4 * dim, S, dim, 1e-6)
            ref.iris_dev_linear_bf16(h, norm, w_in.data_ptr(), S, dim, ldh)
            ref.iris_dev_head_norm_rope(h, ldh, nq.data_ptr(), d_cos, d_sin, S, H, D, 1e-6, 0)
            ref.iris_dev_head_norm_rope(h + 2 * dim, ldh, nk.data_ptr(), d_cos, d_sin, S, H, D, 1e-6, 0)
            ref.iris_dev_attention(cat, ldc, h, h + 2 * dim, h + 4 * dim, ldh, S, S, H, H, D, 1.0 / np.sqrt(D), 0, None)
            ref.iris_dev_swiglu(cat + 2 * dim, ldc, h + 6 * dim, h + 2 * (3 * dim + mlp), ldh, S, mlp)
            ref.iris_dev_linear_f32(proj.data_ptr(), cat, w_out.data_ptr(), S, ldc, dim)
            ref.iris_dev_residual(xr.data_ptr(), proj.data_ptr(), mod.data_ptr() + 8 * dim, S, dim)

        for _ in range(2):
            theirs()
        ref.iris_dev_sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            theirs()
        ref.iris_dev_sync()
        rms = (time.perf_counter() - t0) * 1e3 / reps
        out["reference_cuda_ms"] = round(rms, 4)
        out["reference_cuda"] = "iris_cuda.cu unmodified, -arch=sm_100: cuBLAS GEMMs + its own kernels, 8 calls"
        out["speedup_vs_reference_cuda"] = round(rms / ms, 3)
    for p in (d_cos, d_sin, scratch):
        lib.iris_dev_free(p)
    return out


def double_block_run(job, w, pk, reps=10):
    """One double-stream block (rank 0, N = 1): seven launches through
    iris_b200_double_block next to the reference's CUDA backend issuing its
    twenty-seven calls (iris_transformer_flux.c:3781-3823) on the same device."""
    lib, torch = job.lib, job.torch
    import ctypes as C
    binding = sys.modules[type(lib).__module__]
    S, H, T = seq_len(w), w["heads"], w["txt"]
    dim, mlp = H * D, 3 * H * D
    gen = torch.Generator(device="cuda").manual_seed(13)

    def rnd(shape, scale=1.0, dtype=torch.float32):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * scale).to(dtype)

    x0 = rnd((S, dim))
    x = x0.clone()
    keep, streams = [], []
    for _ in range(2):
        t = dict(qkv=rnd((3 * dim, dim), dim ** -0.5, torch.bfloat16), proj=rnd((dim, dim), dim ** -0.5, torch.bfloat16),
                 ff_in=rnd((2 * mlp, dim), dim ** -0.5, torch.bfloat16), ff_out=rnd((dim, mlp), mlp ** -0.5, torch.bfloat16),
                 norm_q=1 + 0.1 * rnd((D,)), norm_k=1 + 0.1 * rnd((D,)), mod=rnd((6 * dim,), 0.3))
        keep.append(t)
        streams.append(binding.StreamWeights(*[t[k].data_ptr() for k in
                                               ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k", "mod")]))
    cos, sin = rope_tables(w)
    d_cos, d_sin = lib.to_device(cos), lib.to_device(sin)
    scratch = lib.alloc(lib.iris_b200_double_block_scratch_bytes(S, dim, mlp))
    torch.cuda.synchronize()

    def ours():
        rc = lib.iris_b200_double_block(x.data_ptr(), scratch, C.addressof(streams[0]), C.addressof(streams[1]), d_cos,
                                        d_sin, S, T, dim, H, mlp, None)
        assert rc == 0, rc

    for _ in range(3):
        ours()
    lib.iris_dev_sync()
    n0 = lib.iris_b200_launch_count()
    lib.iris_b200_mark(0)
    for _ in range(reps):
        ours()
    lib.iris_b200_mark(1)
    ms = lib.iris_b200_mark_elapsed_ms(0, 1) / reps
    launches = (lib.iris_b200_launch_count() - n0) // reps
    lib.check()
    flops = 2.0 * S * dim * 3 * dim + 4.0 * S * S * dim + 2.0 * S * dim * dim + 2.0 * S * dim * 2 * mlp + 2.0 * S * mlp * dim
    out = {"shape": {"tokens": S, "text": T, "dim": dim, "heads": H, "mlp": mlp}, "launches_per_block": int(launches),
           "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
           "frac_of_bf16_sustained": round(flops / ms / 1e9 / pk[1], 4)}
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    ref = ol.ref_cuda()
    if ref is not None and ref.iris_dev_init() == 1:
        ldh = max(3 * dim, 2 * mlp)
        r_norm = torch.empty((S, dim), device="cuda", dtype=torch.bfloat16)
        r_h = torch.empty((S, ldh), device="cuda", dtype=torch.bfloat16)
        r_cat = torch.empty((S, max(dim, mlp)), device="cuda", dtype=torch.bfloat16)
        norm, h, cat = r_norm.data_ptr(), r_h.data_ptr(), r_cat.data_ptr()
        proj = torch.empty((S, dim), device="cuda", dtype=torch.float32)
        xr = x0.clone()
        torch.cuda.synchronize()

        def theirs():
            for m in range(2):
                t, n, first = keep[m], (S - T) if m else T, T if m else 0
                mod, xo, qkv = t["mod"].data_ptr(), xr.data_ptr() + first * dim * 4, h + 3 * first * dim * 2
                ref.iris_dev_layer_norm_mod(norm, xo, mod, mod + 4 * dim, n, dim, 1e-6)
                ref.iris_dev_linear_bf16(qkv, norm, t["qkv"].data_ptr(), n, dim, 3 * dim)
                ref.iris_dev_head_norm_rope(qkv, 3 * dim, t["norm_q"].data_ptr(), d_cos + first * 64 * 4,
                                            d_sin + first * 64 * 4, n, H, D, 1e-6, 0)
                ref.iris_dev_head_norm_rope(qkv + 2 * dim, 3 * dim, t["norm_k"].data_ptr(), d_cos + first * 64 * 4,
                                            d_sin + first * 64 * 4, n, H, D, 1e-6, 0)
            ref.iris_dev_attention(cat, dim, h, h + 2 * dim, h + 4 * dim, 3 * dim, S, S, H, H, D, 1.0 / np.sqrt(D), 0, None)
            for m in range(2):
                t, n, first = keep[m], (S - T) if m else T, T if m else 0
                mod, xo = t["mod"].data_ptr(), xr.data_ptr() + first * dim * 4
                ref.iris_dev_linear_f32(proj.data_ptr(), cat + first * dim * 2, t["proj"].data_ptr(), n, dim, dim)
                ref.iris_dev_residual(xo, proj.data_ptr(), mod + 8 * dim, n, dim)
            for m in range(2):
                t, n, first = keep[m], (S - T) if m else T, T if m else 0
                mod, xo = t["mod"].data_ptr(), xr.data_ptr() + first * dim * 4
                ref.iris_dev_layer_norm_mod(norm, xo, mod + 12 * dim, mod + 16 * dim, n, dim, 1e-6)
                ref.iris_dev_linear_bf16(h, norm, t["ff_in"].data_ptr(), n, dim, 2 * mlp)
                ref.iris_dev_swiglu(cat, mlp, h, h + 2 * mlp, 2 * mlp, n, mlp)
                ref.iris_dev_linear_f32(proj.data_ptr(), cat, t["ff_out"].data_ptr(), n, mlp, dim)
                ref.iris_dev_residual(xo, proj.data_ptr(), mod + 20 * dim, n, dim)

        for _ in range(2):
            theirs()
        ref.iris_dev_sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            theirs()
        ref.iris_dev_sync()
        rms = (time.perf_counter() - t0) * 1e3 / reps
        out["reference_cuda_ms"] = round(rms, 4)
        out["speedup_vs_reference_cuda"] = round(rms / ms, 3)
    for p in (d_cos, d_sin, scratch):
        lib.iris_dev_free(p)
    return out


def other_blocks_run(job, pk, reps=6):
    """One Z-Image block (config 4: 4608 padded rows, dim 3840, ff 10240) and one
    FLUX.3 block over the multi-reference sequence (config 5: 16 896 rows in
    three segments, dim 3072, mlp 9216) through iris_b200_zimage_block and
    iris_b200_single_block_segments, each next to the reference's CUDA backend
    issuing its own calls (iris_transformer_zimage.c:1940-1959,
    iris_transformer_flux3.c:680-703) on the same device (rank 0, N = 1)."""
    lib, torch = job.lib, job.torch
    import ctypes as C
    binding = sys.modules[type(lib).__module__]
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    ref = ol.ref_cuda()
    if ref is not None and ref.iris_dev_init() != 1:
        ref = None
    gen = torch.Generator(device="cuda").manual_seed(17)

    def rnd(shape, scale=1.0, dtype=torch.float32):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * scale).to(dtype)

    def timed(fn, sync):
        for _ in range(2):
            fn()
        sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        sync()
        return (time.perf_counter() - t0) * 1e3 / reps

    def ours_ms(fn):
        for _ in range(2):
            fn()
        lib.iris_dev_sync()
        lib.iris_b200_mark(0)
        for _ in range(reps):
            fn()
        lib.iris_b200_mark(1)
        ms = lib.iris_b200_mark_elapsed_ms(0, 1) / reps
        lib.check()
        return ms

    out = {}
    # ---- Z-Image ----
    w = WORKLOADS["zimage-turbo"]
    S, H = seq_len(w), w["heads"]
    dim, ff = H * D, 10240
    cos, sin = rope_tables(w)
    d_cos, d_sin = lib.to_device(cos), lib.to_device(sin)
    x = rnd((S, dim))
    t = dict(qkv=rnd((3 * dim, dim), dim ** -0.5, torch.bfloat16), proj=rnd((dim, dim), dim ** -0.5, torch.bfloat16),
             ff_in=rnd((2 * ff, dim), dim ** -0.5, torch.bfloat16), ff_out=rnd((dim, ff), ff ** -0.5, torch.bfloat16),
             norm_q=1 + 0.1 * rnd((D,)), norm_k=1 + 0.1 * rnd((D,)))
    norms = [1 + 0.1 * rnd((dim,)) for _ in range(4)]
    mod = rnd((4 * dim,), 0.3)
    wz = binding.ZImageWeights(*[t[k].data_ptr() for k in ("qkv", "proj", "ff_in", "ff_out", "norm_q", "norm_k")],
                               *[n.data_ptr() for n in norms])
    scratch = lib.alloc(lib.iris_b200_zimage_block_scratch_bytes(S, dim, ff))
    torch.cuda.synchronize()

    def zi():
        rc = lib.iris_b200_zimage_block(x.data_ptr(), scratch, C.addressof(wz), mod.data_ptr(), d_cos, d_sin, S, dim, H, ff, None)
        assert rc == 0, rc

    n0 = lib.iris_b200_launch_count()
    ms = ours_ms(zi)
    launches = (lib.iris_b200_launch_count() - n0) // (reps + 2)
    flops = 2.0 * S * dim * (3 * dim + dim + 2 * ff + ff) + 4.0 * S * S * dim
    z = {"shape": {"tokens": S, "dim": dim, "heads": H, "ff": ff}, "launches_per_block": int(launches), "ms": round(ms, 4),
         "tflops": round(flops / ms / 1e9, 1), "frac_of_bf16_sustained": round(flops / ms / 1e9 / pk[1], 4)}
    if ref is not None:
        norm = torch.empty((S, dim), device="cuda", dtype=torch.bfloat16).data_ptr()
        r_h = torch.empty((S, max(3 * dim, 2 * ff)), device="cuda", dtype=torch.bfloat16)
        r_act = torch.empty((S, max(dim, ff)), device="cuda", dtype=torch.bfloat16)
        r_out = torch.empty((S, dim), device="cuda", dtype=torch.float32)
        h, act, o, xp, m = r_h.data_ptr(), r_act.data_ptr(), r_out.data_ptr(), x.data_ptr(), mod.data_ptr()

        def zi_ref():
            ref.iris_dev_rms_norm_mod(norm, xp, norms[0].data_ptr(), m, S, dim, 1e-5)
            ref.iris_dev_linear_bf16(h, norm, t["qkv"].data_ptr(), S, dim, 3 * dim)
            ref.iris_dev_head_norm_rope(h, 3 * dim, t["norm_q"].data_ptr(), d_cos, d_sin, S, H, D, 1e-5, 0)
            ref.iris_dev_head_norm_rope(h + 2 * dim, 3 * dim, t["norm_k"].data_ptr(), d_cos, d_sin, S, H, D, 1e-5, 0)
            ref.iris_dev_attention(act, dim, h, h + 2 * dim, h + 4 * dim, 3 * dim, S, S, H, H, D, 1.0 / np.sqrt(D), 0, None)
            ref.iris_dev_linear_f32(o, act, t["proj"].data_ptr(), S, dim, dim)
            ref.iris_dev_rms_norm_residual(xp, o, norms[1].data_ptr(), m + 4 * dim, S, dim, 1e-5)
            ref.iris_dev_rms_norm_mod(norm, xp, norms[2].data_ptr(), m + 8 * dim, S, dim, 1e-5)
            ref.iris_dev_linear_bf16(h, norm, t["ff_in"].data_ptr(), S, dim, 2 * ff)
            ref.iris_dev_swiglu(act, ff, h, h + 2 * ff, 2 * ff, S, ff)
            ref.iris_dev_linear_f32(o, act, t["ff_out"].data_ptr(), S, ff, dim)
            ref.iris_dev_rms_norm_residual(xp, o, norms[3].data_ptr(), m + 12 * dim, S, dim, 1e-5)

        lib.iris_dev_sync()
        rms = timed(zi_ref, ref.iris_dev_sync)
        z["reference_cuda_ms"] = round(rms, 4)
        z["speedup_vs_reference_cuda"] = round(rms / ms, 3)
        del r_h, r_act, r_out
    for p in (d_cos, d_sin, scratch):
        lib.iris_dev_free(p)
    del x, t, norms
    out["zimage_block"] = z
    # ---- FLUX.3, three segments ----
    w = WORKLOADS["flux3-multiref"]
    S, H = seq_len(w), w["heads"]
    dim, mlp = H * D, 3 * H * D
    ldh, ldc = 3 * dim + 2 * mlp, dim + mlp
    cos, sin = rope_tables(w)
    d_cos, d_sin = lib.to_device(cos), lib.to_device(sin)
    x = rnd((S, dim))
    w_in, w_out = rnd((ldh, dim), dim ** -0.5, torch.bfloat16), rnd((dim, ldc), ldc ** -0.5, torch.bfloat16)
    nq, nk = 1 + 0.1 * rnd((D,)), 1 + 0.1 * rnd((D,))
    img = w["img"][0] * w["img"][1]
    lens = [w["txt"], img, S - w["txt"] - img]
    mods = [rnd((3 * dim,), 0.3) for _ in lens]
    segs = (binding.Segment * 3)(*[binding.Segment(int(sum(lens[:i])), int(n), mods[i].data_ptr()) for i, n in enumerate(lens)])
    scratch = lib.alloc(lib.iris_b200_single_block_scratch_bytes(S, dim, mlp))
    torch.cuda.synchronize()

    def f3():
        rc = lib.iris_b200_single_block_segments(x.data_ptr(), scratch, w_in.data_ptr(), w_out.data_ptr(), nq.data_ptr(),
                                                 nk.data_ptr(), C.addressof(segs), 3, d_cos, d_sin, S, dim, H, mlp, 1e-6, None)
        assert rc == 0, rc

    ms = ours_ms(f3)
    flops = 2.0 * S * dim * ldh + 4.0 * S * S * dim + 2.0 * S * ldc * dim
    f = {"shape": {"tokens": S, "segments": lens, "dim": dim, "heads": H, "mlp": mlp}, "launches_per_block": 4,
         "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_of_bf16_sustained": round(flops / ms / 1e9 / pk[1], 4)}
    if ref is not None:
        norm = torch.empty((S, dim), device="cuda", dtype=torch.bfloat16)
        r_h = torch.empty((S, ldh), device="cuda", dtype=torch.bfloat16)
        r_cat = torch.empty((S, ldc), device="cuda", dtype=torch.bfloat16)
        r_out = torch.empty((S, dim), device="cuda", dtype=torch.float32)
        nr, h, cat, o, xp = norm.data_ptr(), r_h.data_ptr(), r_cat.data_ptr(), r_out.data_ptr(), x.data_ptr()

        def f3_ref():
            for i, n in enumerate(lens):
                off = int(sum(lens[:i])) * dim
                m = mods[i].data_ptr()
                ref.iris_dev_layer_norm_mod(nr + off * 2, xp + off * 4, m, m + 4 * dim, n, dim, 1e-6)
            ref.iris_dev_linear_bf16(h, nr, w_in.data_ptr(), S, dim, ldh)
            ref.iris_dev_head_norm_rope(h, ldh, nq.data_ptr(), d_cos, d_sin, S, H, D, 1e-6, 0)
            ref.iris_dev_head_norm_rope(h + 2 * dim, ldh, nk.data_ptr(), d_cos, d_sin, S, H, D, 1e-6, 0)
            ref.iris_dev_attention(cat, ldc, h, h + 2 * dim, h + 4 * dim, ldh, S, S, H, H, D, 1.0 / np.sqrt(D), 0, None)
            ref.iris_dev_swiglu(cat + 2 * dim, ldc, h + 6 * dim, h + 2 * (3 * dim + mlp), ldh, S, mlp)
            ref.iris_dev_linear_f32(o, cat, w_out.data_ptr(), S, ldc, dim)
            for i, n in enumerate(lens):
                off = int(sum(lens[:i])) * dim
                ref.iris_dev_residual(xp + off * 4, o + off * 4, mods[i].data_ptr() + 8 * dim, n, dim)

        lib.iris_dev_sync()
        rms = timed(f3_ref, ref.iris_dev_sync)
        f["reference_cuda_ms"] = round(rms, 4)
        f["speedup_vs_reference_cuda"] = round(rms / ms, 3)
    for p in (d_cos, d_sin, scratch):
        lib.iris_dev_free(p)
    out["flux3_block"] = f
    return out


def outproj_run(job, pk, reps=20):
    """The step after the path with the heads sharded over the ranks (N > 1):
    the Klein-4B block's out-projection, [4608, dim / N] x [dim, dim / N]^T per
    rank, whose fp32 partial sums are reduced across the ranks by the GEMM's
    epilogue (stores over NVLink to the rows' owners) and folded into the
    gated residual on the owner. Needs the group of the ring."""
    lib, torch, rank, world = job.lib, job.torch, job.rank, job.world
    w = WORKLOADS["klein4b-1024"]
    S, dim = seq_len(w), w["heads"] * D
    a, b = C.c_int(), C.c_int()
    rows_of = np.zeros(world, np.int32)
    for r in range(world):
        lib.iris_b200_seq_shard(S, world, r, C.byref(a), C.byref(b))
        rows_of[r] = b.value
    lib.iris_b200_head_shard(w["heads"], world, rank, C.byref(a), C.byref(b))
    k0, k = a.value * D, b.value * D
    gen = torch.Generator(device="cuda").manual_seed(9 + rank)
    cat = torch.randn((S, k), generator=gen, device="cuda").to(torch.bfloat16)
    W = (torch.randn((dim, dim), generator=gen, device="cuda") / dim ** 0.5).to(torch.bfloat16)
    x = torch.zeros((int(rows_of[rank]), dim), device="cuda", dtype=torch.float32)
    gate = torch.ones(dim, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()

    def call():
        rc = lib.iris_b200_outproj_residual(x.data_ptr(), cat.data_ptr(), k, W.data_ptr() + k0 * 2, dim, gate.data_ptr(),
                                            rows_of.ctypes.data, k, dim)
        assert rc == 0, rc

    for _ in range(3):
        call()
    job.barrier()
    lib.iris_b200_mark(0)
    for _ in range(reps):
        call()
    lib.iris_b200_mark(1)
    job.barrier()
    ms = job.max_over_ranks([lib.iris_b200_mark_elapsed_ms(0, 1) / reps])[0]
    lib.check()
    # The library sequence on the same operands: cuBLAS GEMM (bf16 result, which
    # rounds the partial sums the fused kernel keeps in fp32), widened, NCCL
    # reduce-scatter, residual. Equal row counts only.
    lib_ms = None
    if len(set(int(r) for r in rows_of)) == 1:
        Wk = W[:, k0:k0 + k]
        part = torch.empty((S, dim), device="cuda", dtype=torch.float32)
        own = torch.empty((int(rows_of[rank]), dim), device="cuda", dtype=torch.float32)

        def lib_call():
            part.copy_(torch.matmul(cat, Wk.t()))
            job.dist.reduce_scatter_tensor(own, part)
            x.addcmul_(own, gate)

        for _ in range(3):
            lib_call()
        job.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            lib_call()
        e1.record()
        job.barrier()
        lib_ms = job.max_over_ranks([e0.elapsed_time(e1) / reps])[0]
    sent = float(S - rows_of[rank]) * dim * 4
    return {"shape": [S, dim // world, dim], "ms": round(ms, 4),
            "cublas_nccl_reduce_scatter_residual_ms": round(lib_ms, 4) if lib_ms else None,
            "what": "GEMM + reduce-scatter in its epilogue (peer stores) + gated residual on the owner",
            "gemm_tflops_aggregate": round(2.0 * S * dim * dim / ms / 1e9, 1),
            "nvlink_bytes_per_rank": sent, "nvlink_gbs_per_rank": round(sent / ms / 1e6, 1)}


def tp_block_run(job, pk, reps=10):
    """One Klein-4B single-stream block, tensor parallel over the ranks (N > 1):
    rows of the hidden state owned by the ranks, heads and MLP columns sharded;
    the all-gather lives in the LayerNorm's stores and the projection's arrival
    waits, the reduce-scatter in the output projection's epilogue
    (iris_b200_single_block_tp). Needs the group of the ring. ms per block, max
    over ranks; the one-GPU block is `single_block` of the N = 1 line."""
    lib, torch, rank, world = job.lib, job.torch, job.rank, job.world
    w = WORKLOADS["klein4b-1024"]
    S, H = seq_len(w), w["heads"]
    dim, mlp = H * D, 3 * H * D
    if H % world or mlp % (8 * world):
        return None
    hl, ml = H // world, mlp // world
    a, b = C.c_int(), C.c_int()
    rows_of = np.zeros(world, np.int32)
    for r in range(world):
        lib.iris_b200_seq_shard(S, world, r, C.byref(a), C.byref(b))
        rows_of[r] = b.value
    gen = torch.Generator(device="cuda").manual_seed(21 + rank)

    def rnd(shape, scale=1.0, dtype=torch.float32):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * scale).to(dtype)

    x = rnd((int(rows_of[rank]), dim))
    w_in = rnd((3 * hl * D + 2 * ml, dim), dim ** -0.5, torch.bfloat16)
    w_out = rnd((dim, hl * D + ml), (dim + mlp) ** -0.5, torch.bfloat16)
    nq, nk, mod = 1 + 0.1 * rnd((D,)), 1 + 0.1 * rnd((D,)), rnd((3 * dim,), 0.3)
    cos, sin = rope_tables(w)
    d_cos, d_sin = lib.to_device(cos), lib.to_device(sin)
    scratch = lib.alloc(lib.iris_b200_single_block_tp_scratch_bytes(S, hl, ml))
    torch.cuda.synchronize()

    def call():
        rc = lib.iris_b200_single_block_tp(x.data_ptr(), scratch, w_in.data_ptr(), w_out.data_ptr(), nq.data_ptr(),
                                           nk.data_ptr(), mod.data_ptr(), d_cos, d_sin, rows_of.ctypes.data, dim, hl, ml, None)
        assert rc == 0, rc

    # every rank tries three blocks; the timed part only runs when all of them got through
    ok, why = 1, ""
    try:
        for _ in range(3):
            call()
        lib.iris_dev_sync()
        lib.check()
    except Exception as e:
        ok, why = 0, repr(e)[:160]
    flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
    job.dist.all_reduce(flag, op=job.dist.ReduceOp.MIN)
    if int(flag.item()) == 0:
        lib.iris_b200_clear_error()
        return {"error": why or "another rank failed"}
    job.barrier()
    lib.iris_b200_mark(0)
    for _ in range(reps):
        call()
    lib.iris_b200_mark(1)
    job.barrier()
    ms = job.max_over_ranks([lib.iris_b200_mark_elapsed_ms(0, 1) / reps])[0]
    lib.check()
    for p in (d_cos, d_sin, scratch):
        lib.iris_dev_free(p)
    flops = 2.0 * S * dim * (3 * dim + 2 * mlp) + 4.0 * S * S * dim + 2.0 * S * (dim + mlp) * dim
    return {"shape": {"tokens": S, "dim": dim, "heads_per_rank": hl, "mlp_per_rank": ml}, "ms": round(ms, 4),
            "tflops": round(flops / ms / 1e9, 1), "per_gpu_pct_bf16_sustained": round(100 * flops / ms / 1e9 / world / pk[1], 2),
            "gathered_bytes_per_rank": int((S - int(rows_of[rank])) * dim * 2),
            "scattered_bytes_per_rank": int((S - int(rows_of[rank])) * dim * 4)}


def extra_run(job, name, mode, steps, warmup, pk, groups=1):
    """A further workload / decomposition measured in the same run: ms per
    step (max over ranks), aggregate TFLOP/s and per-GPU share of the peak."""
    w = WORKLOADS[name]
    plan = plan_of(job, w, mode, groups)
    B = Buffers(job, w, plan)
    res = timed_steps(job, w, plan, B, steps, warmup, marks=(job.rank == 0))
    B.free()
    total = attn_flops(w["batch"], w["heads"], plan["S_full"], plan["S_full"]) / (res["ms"] * 1e-3) / 1e12
    out = {"workload": name, "mode": mode, "ms_per_step": round(res["ms"], 4), "tflops": round(total, 1),
           "per_gpu_pct_bf16_peak": round(100 * total / job.world / pk[0], 2)}
    if res.get("attn_ms"):
        # rank 0's own launches (one batch entry per rank): what a step spends outside the attention kernel
        kms, pms = float(np.mean(res["attn_ms"])), float(np.mean(res["pro_ms"])) if res.get("pro_ms") else None
        out["rank0_attention_kernel_ms"] = round(kms, 4)
        out["rank0_prologue_ms"] = round(pms, 4) if pms else None
    return out


def ring_extra_run(job, name, steps, warmup, pk, groups, parts):
    """A further ring decomposition of the same workload (`groups` head groups
    x rings of world / groups): the rings are set up afresh, every rank tries
    two steps, and only when all of them got through is it measured - a side
    measurement must not cost the headline line."""
    torch, lib = job.torch, job.lib
    w = WORKLOADS[name]
    ok, why = 1, ""
    try:
        lib.iris_b200_ring_destroy()        # whatever state an earlier attempt left behind
        job.ring_ready = False
        job.ring_init(parts, groups)
        plan = plan_of(job, w, "ring", groups)
        B = Buffers(job, w, plan)
        try:
            for _ in range(2):
                run_step(job, w, plan, B, B.sets[0])
            lib.iris_dev_sync()
            lib.check()
        finally:
            B.free()
    except Exception as e:
        ok, why = 0, repr(e)[:160]
    flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
    job.dist.all_reduce(flag, op=job.dist.ReduceOp.MIN)
    if int(flag.item()) == 0:
        lib.iris_b200_clear_error()
        return {"error": why or "another rank failed its first steps"}
    return extra_run(job, name, "ring", steps, warmup, pk, groups=groups)


def run_b200(args):
    job = Job()
    lib, torch, rank, world = job.lib, job.torch, job.rank, job.world
    mode = args.mode or ("single" if world == 1 else "ring")
    name = args.workload or ("klein4b-1024" if world == 1 else "flux3-multiref" if mode == "ring" else "klein9b-cfg")
    w = WORKLOADS[name]
    pk = peaks()
    groups, fallback = 1, None
    if mode == "ring":
        # default: rings of two (each rank exchanges K/V rows with one partner: one push per call and a receiver
        # with a single sender), the heads split over world / 2 such rings
        groups = args.head_groups if args.head_groups else (
            world // 2 if world >= 4 and world % 2 == 0 and w["heads"] % (world // 2) == 0 else 1)
    plan = B = None
    if mode == "ring" and groups > 1:
        # Head groups x rings: every rank tries two steps; unless all of them got through, all of them go back
        # to ONE ring over all ranks (the decomposition every multi-GPU test covers).
        ok, why = 1, ""
        try:
            job.ring_init(args.ring_parts, groups)
            plan = plan_of(job, w, mode, groups)
            B = Buffers(job, w, plan)
            for _ in range(2):
                run_step(job, w, plan, B, B.sets[0])
            lib.iris_dev_sync()
            lib.check()
        except Exception as e:
            ok, why = 0, repr(e)[:160]
        flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
        job.dist.all_reduce(flag, op=job.dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            fallback = "head groups failed on some rank (%s): one ring over all ranks instead" % (why or "another rank")
            try:
                if B is not None:
                    B.free()
                lib.iris_b200_clear_error()
                lib.iris_b200_ring_destroy()        # also when ring_init itself got only part of the way
            except Exception:
                pass
            job.ring_ready = False
            groups, plan, B = 1, None, None
    if mode == "ring" and plan is None:
        job.ring_init(args.ring_parts, groups)
    if plan is None:
        plan = plan_of(job, w, mode, groups)
        B = Buffers(job, w, plan)
    S_full, H = plan["S_full"], w["heads"]

    sampler = ClockSampler(job.local) if rank == 0 else None
    res = timed_steps(job, w, plan, B, args.steps, args.warmup, marks=(rank == 0))
    clocks = sampler.stop(*res["wall"]) if sampler else None
    ms_step = res["ms"]
    total_flops = attn_flops(w["batch"], H, S_full, S_full)
    value = total_flops / (ms_step * 1e-3) / 1e12
    roof, prologue = roofline_of(res, name, plan["nh"], plan["S"], S_full, pk) if rank == 0 else (None, None)
    if roof and mode == "ring":
        roof["kernel"] = "k_attention_sm100 (one launch per ring call; the time includes its waits for arriving chunks)"

    e2e = None
    if not args.no_e2e:
        e_ms, serial_ms, h2d, d2h = e2e_steps(job, w, plan, B, args.steps)
        if e_ms > 0:
            e2e = {"value": round(total_flops / (e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(e_ms, 3),
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "how": "iris_b200_upload_async / download_async on two copy streams, ordered by events over 3 "
                          "buffer sets: copies overlap the neighbouring steps",
                   "serial": {"value": round(total_flops / (serial_ms * 1e-3) / 1e12, 2), "ms_per_step": round(serial_ms, 3),
                              "how": "blocking iris_dev_upload / iris_dev_download around every step"}}

    # The GPU result on the uploaded inputs, for the parity check against the CPU leg.
    got = gpu_result(job, w, plan, B)
    host_inputs = B.host_qkv[0] if B.host_qkv else None
    width = B.width
    B.free()

    # Further decompositions in the same run (N > 1 only).
    extras, one_gpu, speedup, group_ok = {}, None, None, True
    if world > 1 and not args.no_extras:
        if mode == "ring":
            # the same workload on ONE GPU (rank 0 alone; the others wait at the barrier)
            if rank == 0:
                p1 = plan_of(job, w, "single")
                B1 = Buffers(job, w, p1)
                r1 = timed_steps(job, w, p1, B1, max(5, min(args.steps, 20)), 3, collective=False)
                B1.free()
                one_gpu = r1["ms"]
            job.barrier()
            one_gpu = job.max_over_ranks([one_gpu or 0.0])[0]
            speedup = one_gpu / ms_step
            if groups > 1:
                # other splits of the same workload: fewer or more head groups (longer or shorter rings), then
                # ONE ring over all ranks with every rank holding all heads
                for g2 in (2, 4):
                    if g2 != groups and world % g2 == 0 and world // g2 >= 2 and H % g2 == 0:
                        extras[name + " %d head groups x rings of %d" % (g2, world // g2)] = ring_extra_run(
                            job, name, args.steps, args.warmup, pk, g2, args.ring_parts)
                one = ring_extra_run(job, name, args.steps, args.warmup, pk, 1, args.ring_parts)
                extras[name + " one ring, all heads per rank"] = one
                group_ok = "error" not in one           # the out-projection and the block below need this group
            extras[name + " head-parallel"] = extra_run(job, name, "shard", args.steps, args.warmup, pk)
        for other in ("klein9b-cfg", "zimage-turbo"):
            if other != name:
                extras[other] = extra_run(job, other, "shard", args.steps, args.warmup, pk)
        if mode == "ring" and not args.no_outproj and group_ok:
            extras["klein4b-1024 out-projection, heads sharded"] = outproj_run(job, pk)
            extras["klein4b-1024 single block, tensor parallel"] = tp_block_run(job, pk)

    # CPU leg on the same inputs (rank 0), and the parity of the two results.
    cpu = parity = ref_gpu = None
    if not args.no_cpu:
        cpu, parity = cpu_leg_with_parity(job, w, plan, got, host_inputs, width, budget_s=20.0 if world == 1 else 12.0)
    if rank == 0 and world == 1 and mode == "single" and not args.no_ref_gpu:
        plan2 = plan_of(job, w, "single")
        B2 = Buffers(job, w, plan2)
        try:
            ref_gpu = reference_gpu_kernels(lib, w, B2.sets[0][0], (B2.d_w, B2.d_cos, B2.d_sin), plan2["S"], plan2["nh"],
                                            1.0 / np.sqrt(D))
        except Exception as e:
            ref_gpu = {"error": repr(e)[:200]}
        B2.free()
    job.ring_destroy()
    projection = None
    if rank == 0 and world == 1 and mode == "single" and w["family"] != "zimage" and not args.no_extras:
        try:
            projection = projection_run(job, w, pk)
        except Exception as e:                     # a side measurement must not cost the headline line
            projection = {"error": repr(e)[:200]}

    block = dblock = others = None
    if rank == 0 and world == 1 and mode == "single" and w["family"] == "flux2" and not args.no_extras:
        try:
            block = block_run(job, w, pk)
        except Exception as e:
            block = {"error": repr(e)[:200]}
        try:
            dblock = double_block_run(job, w, pk)
        except Exception as e:
            dblock = {"error": repr(e)[:200]}
        try:
            others = other_blocks_run(job, pk)
        except Exception as e:
            others = {"error": repr(e)[:200]}

    if rank == 0:
        sharding = {"single": "none",
                    "ring": ("ring sequence parallel" if groups == 1 else
                             "%d head groups x ring sequence parallel over %d GPUs each" % (groups, world // groups)) +
                            ": K/V rows pushed peer to peer by the copy engines, one attention launch per GPU waits "
                            "for them in the kernel; NCCL for set-up",
                    "shard": "cfg batch x heads, no collective"}[mode]
        out = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "batch": w["batch"], "heads": H, "head_dim": D, "tokens": S_full,
                       "step": STEP_WORDS},
            "sharding": sharding if not fallback else sharding + " [" + fallback + "]",
            "l2": "inputs rotate over %d buffer sets (%.0f MB)" % (B.nsets, B.nsets * B.per_set / 1e6),
            "per_gpu_tflops": round(value / world, 2),
            "host_enqueue_ms_per_step": round(res["enqueue_ms"], 4),
            "pct_bf16_peak": round(100 * value / world / pk[0], 2),
            "pct_bf16_sustained": round(100 * value / world / pk[1], 2),
            "clocks": clocks, "e2e": e2e, "gpu_launches": res["launches"],
            "roofline": roof, "roofline_prologue": prologue, "cpu_baseline": cpu, "parity": parity,
            "reference_gpu": ref_gpu, "qkv_projection": projection, "single_block": block,
            "double_block": dblock, "other_blocks": others,
        }
        if speedup is not None:
            out["one_gpu_ms_per_step"] = round(one_gpu, 4)
            out["speedup_vs_1gpu"] = round(speedup, 3)
        if extras:
            out["shards"] = extras
        print(json.dumps(out))
    if job.dist:
        job.dist.destroy_process_group()


def cpu_leg_with_parity(job, w, plan, got, host_inputs, width, budget_s):
    """Rank 0 times the reference's CPU code on the tensors the GPU arm used
    (batch entry 0, the first heads, as many as the time budget allows) and
    compares the two results on every row of those heads."""
    torch, rank, world = job.torch, job.rank, job.world
    S_full, H = plan["S_full"], w["heads"]
    mode = plan["mode"]
    cpu = parity = None
    if mode == "shard" and world > 1:
        return None, None                 # shards of the heads: no parity leg in that mode
    # Assemble the full-sequence inputs on rank 0. In ring mode the other
    # ranks' rows are regenerated from their seeds (seed = 1000 * rank).
    if rank == 0:
        if mode == "ring" and world > 1:
            blocks = [host_inputs] + [make_qkv(int(n), width, 1000 * r) for r, n in enumerate(plan["rows_of"]) if r > 0]
            full = torch.cat([b.cpu() for b in blocks], 0)
        else:
            full = host_inputs

        def inputs(hs):
            n = hs * D
            return tuple(np.ascontiguousarray(bf16_to_f32(full[:, i * width:i * width + n])) for i in range(3))

        r = cpu_reference(w, budget_s=budget_s, steps=1, warmup=0, inputs=inputs, max_heads=width // D)
        cpu, hs, want = r["cpu_baseline"], r["heads_sampled"], r["out"]
    else:
        hs, want = 0, None
    if world > 1:
        t = torch.tensor([hs], device="cuda")
        job.dist.broadcast(t, src=0)
        hs = int(t.item())
        # every rank's rows of the compared heads -> rank 0
        mine = got[:, :hs * D].contiguous().cuda()
        rows_max = int(max(plan["rows_of"]))
        pad = torch.zeros((rows_max, hs * D), dtype=torch.bfloat16, device="cuda")
        pad[:mine.shape[0]] = mine
        gathered = [torch.empty_like(pad) for _ in range(world)] if rank == 0 else None
        job.dist.gather(pad, gathered, dst=0)
        if rank == 0:
            # rank 0's ring is the ranks [0, ring size): their rows, in order, are the whole sequence
            got_all = torch.cat([gathered[r][:int(n)].cpu() for r, n in enumerate(plan["rows_of"])], 0)
    else:
        got_all = got[:, :hs * D]
    if rank == 0:
        mx, cs = head_errors(bf16_to_f32(got_all), want, hs)
        parity = {"max_abs": round(mx, 5), "min_cos": round(cs, 7), "heads": hs, "rows": int(S_full),
                  "against": cpu["kind"] + " CPU result on the same bf16-rounded inputs, every row of the compared heads",
                  "tolerance": {"max_abs": 2e-2, "min_cos": 0.9999}, "ok": bool(mx <= 2e-2 and cs >= 0.9999)}
    return cpu, parity


# ---------------------------------------------------------------------------
# the reference arm / CPU baseline (the only part that may execute oracle/)
# ---------------------------------------------------------------------------

def reference_gpu_kernels(lib, w, bufs, consts, S, nh, scale, reps=20):
    """The reference's own CUDA backend (iris_cuda.cu compiled unmodified for
    sm_100 into oracle/_ref) on the same device buffers: its two prologue
    launches and its mma.sync flash attention, timed by wall clock between
    its stream syncs (it has no event API). Context for the B200 numbers:
    what the reference itself achieves on this GPU."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    ref = ol.ref_cuda()
    if ref is None or ref.iris_dev_init() != 1:
        return None
    dq, dout = bufs
    d_w, d_cos, d_sin = consts
    width = nh * D
    q, k, v = dq, dq + width * 2, dq + 2 * width * 2
    lib.iris_dev_sync()

    def attn():
        ref.iris_dev_attention(dout, width, q, k, v, 3 * width, S, S, nh, nh, D, scale, 0, None)

    def pro():
        ref.iris_dev_head_norm_rope(q, 3 * width, d_w, d_cos, d_sin, S, nh, D, w["eps"], 0)
        ref.iris_dev_head_norm_rope(k, 3 * width, d_w, d_cos, d_sin, S, nh, D, w["eps"], 0)

    out = {}
    for name, fn in (("attention_ms", attn), ("prologue_ms", pro)):
        for _ in range(3):
            fn()
        ref.iris_dev_sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        ref.iris_dev_sync()
        out[name] = round((time.perf_counter() - t0) * 1e3 / reps, 4)
    out["attention_tflops"] = round(attn_flops(1, nh, S, S) / (out["attention_ms"] * 1e-3) / 1e12, 1)
    out["kernel"] = "reference k_flash_attention (mma.sync m16n8k16) + k_head_norm_rope x2, -arch=sm_100"
    return out


def cpu_reference(w, budget_s, steps, warmup, inputs=None, max_heads=None):
    """Times the reference's CPU code for one step of workload `w` on the host
    cores: Q/K norm + RoPE, then attention. Uses oracle/_ref (the reference
    sources compiled unmodified: BLAS build if it loads, else generic), else
    the CPU port. The sample is a subset of heads sized to the time budget.
    inputs(hs) -> fp32 (q, k, v) [S, hs * 128] of the first hs heads: the
    tensors of the GPU arm; without it seeded normal values are drawn. The
    result of the last pass comes back as `out` for the parity check."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")
    S, H = seq_len(w), w["heads"]
    ncpu = os.cpu_count() or 1
    ref = ol.ref("blas")
    kind, variant = "reference", "blas: mha_forward, pthreads over heads + cblas_sgemm"
    if ref is not None:
        ref.openblas_set_num_threads(1)
    else:
        ref = ol.ref("generic")
        variant = "generic: iris_flash_attention, 1 thread"
    if ref is None:
        kind, variant = "port", "oracle port: orc_dev_attention, pthreads over heads"
    cos, sin = rope_tables(w)
    cos2, sin2 = np.repeat(cos, 2, axis=1).copy(), np.repeat(sin, 2, axis=1).copy()

    last = {}

    def one(hs):
        if inputs is not None:
            q, k, v = inputs(hs)
        else:
            rng = np.random.default_rng(7)
            q, k, v = (rng.standard_normal((S, hs * D), dtype=np.float32) for _ in range(3))
        ones = np.ones(D, np.float32)
        out = np.zeros_like(q)
        t0 = time.perf_counter()
        if kind == "reference":
            if w["family"] == "flux3":
                ref.ref_f3_head_rms_norm(q, ones, S, hs, D, w["eps"])
                ref.ref_f3_head_rms_norm(k, ones, S, hs, D, w["eps"])
                ref.ref_f3_apply_rope(q, cos, sin, S, hs, D)
                ref.ref_f3_apply_rope(k, cos, sin, S, hs, D)
                assert ref.ref_f3_attention(out, q, k, v, S, hs, D) == 0
            else:
                ref.ref_flux_qk_norm(q, k, ones, ones, S, hs, D, w["eps"])
                ref.ref_flux_apply_rope_2d(q, cos2, sin2, S, hs, D)
                ref.ref_flux_apply_rope_2d(k, cos2, sin2, S, hs, D)
                if "blas" in variant:
                    assert ref.ref_flux_mha(out, q, k, v, S, hs, D) == 0
                else:
                    ref.iris_flash_attention(out, q, k, v, S, S, hs, D, 1.0 / np.sqrt(D))
        else:
            o = ol.oracle()
            o.orc_head_norm_rope_f32(q.ctypes.data, hs * D, ones, cos, sin, S, hs, D, w["eps"], 0)
            o.orc_head_norm_rope_f32(k.ctypes.data, hs * D, ones, cos, sin, S, hs, D, w["eps"], 0)
            out = ol.dev_attention(q, k, v, hs)
        dt = time.perf_counter() - t0
        last["out"] = out
        return dt

    # Head count of the sample. The reference's BLAS build runs one pthread
    # per group of heads (thread count = largest divisor of the head count
    # that fits the cores, fixed at its first call), so samples there are
    # whole multiples of that thread count; its FLUX.3 routine and the
    # generic build walk heads serially. One calibration pass sizes the
    # sample to the time budget, then the timed passes run.
    threads, unit = 1, 1
    H = min(H, max_heads) if max_heads else H          # the inputs at hand may hold fewer heads than the model
    if kind == "reference" and "blas" in variant:
        if w["family"] == "flux3":
            ref.openblas_set_num_threads(ncpu)
            threads = ncpu
            variant = "blas: attention (256-query chunks), OpenBLAS threads"
        else:
            threads = unit = ref.ref_flux_attn_threads(H)
    elif kind == "port":
        threads = unit = min(ncpu, H)
    hs = unit
    t_cal = one(hs)
    per_step_budget = budget_s / max(1, steps + warmup + 1)
    want = int(hs * per_step_budget / max(t_cal, 1e-6)) // unit * unit
    hs = max(unit, min(H // unit * unit if H >= unit else H, want))
    times = []
    for i in range(warmup + steps):
        t = one(hs)
        if i >= warmup:
            times.append(t)
    t = sum(times) / len(times)
    flops = attn_flops(1, hs, S, S)
    val = flops / t / 1e12
    return {"seconds_per_step": t, "value": val, "heads_sampled": hs, "out": last["out"],
            "cpu_baseline": {"value": round(val, 5), "unit": "TFLOP/s", "cores": int(threads), "host_cores": ncpu,
                             "kind": kind, "variant": variant,
                             "sample": "%d of %d heads x %d tokens, batch entry 0, fp32, prologue + attention, %.2f s per pass"
                                       % (hs, H, S, t)}}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return
    mode = args.mode or ("single" if world == 1 else "ring")
    name = args.workload or ("klein4b-1024" if world == 1 else "flux3-multiref" if mode == "ring" else "klein9b-cfg")
    w = WORKLOADS[name]
    r = cpu_reference(w, budget_s=150.0, steps=args.steps, warmup=args.warmup)
    S = seq_len(w)
    out = {
        "impl": "reference",
        "metric": METRIC,
        "value": round(r["value"], 5), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(r["seconds_per_step"] * 1e3, 2), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "batch": w["batch"], "heads": w["heads"], "head_dim": D, "tokens": S,
                   "step": STEP_WORDS},
        "where": "host CPU",
        "cpu_baseline": r["cpu_baseline"],
        "e2e": {"value": round(r["value"], 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffer) measurement")
    ap.add_argument("--mode", default=None, choices=["single", "shard", "ring"],
                    help="N > 1: ring sequence parallelism (default) or independent cfg/head shards")
    ap.add_argument("--head-groups", type=int, default=0,
                    help="ring mode: split the heads over this many independent rings (0: rings of two from four GPUs up, else one ring)")
    ap.add_argument("--ring-parts", type=int, default=0, help="key parts of a ring call's launch (0: the library's choice)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the further measurements of the same run (N > 1: other workloads; N = 1: the QKV projection)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-outproj", action="store_true", help="N > 1: skip the out-projection measurement")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip the reference's own CUDA kernels")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
