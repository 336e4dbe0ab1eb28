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
runs the Klein-9B CFG block (batch 2 x 32 heads x 4608 tokens) with the two
batch entries on disjoint GPU groups and the heads of an entry sharded over
the GPUs of its group: independent shards, no collective in the data path.

Data is synthetic: seeded N(0,1) Q/K/V in bf16, unit norm weights and the
RoPE tables of the model family; the reference publishes no dataset for this
path. Inputs rotate through several buffer sets larger than L2 in total.

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


# dram__bytes_read.sum + dram__bytes_write.sum of one k_attention_sm100 launch, from the ncu capture
# summarised in profiles/k_attention_sm100_klein4b-1024.md (algorithmic Q+K+V+O: 113.2 MB).
NCU_DRAM_BYTES_PER_LAUNCH = {"klein4b-1024": 91.5e6}


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


def shard_of(w, rank, world):
    """(batch entry, first head, head count) of this rank: batch entries on
    disjoint GPU groups, heads of an entry split evenly over its group (the
    first heads % group ranks take one more)."""
    B, H = w["batch"], w["heads"]
    groups = min(B, world)
    per = world // groups
    grp, r = min(rank // per, groups - 1), rank % per
    if rank >= groups * per:           # leftover ranks when world is not a multiple of the batch
        return None
    base, extra = divmod(H, per)
    h0 = r * base + min(r, extra)
    nh = base + (1 if r < extra else 0)
    entries = list(range(grp, B, groups))
    return entries, h0, nh


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p.get("bf16_tflops", 1632.7), p.get("bf16_tflops_sustained", 1365.4), p.get("hbm_gbs", 6551.0), "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


def run_b200(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dist = None
    import torch
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ring = args.mode == "ring"
    name = args.workload or ("flux3-multiref" if ring else "klein4b-1024" if world == 1 else "klein9b-cfg")
    w = WORKLOADS[name]
    lib = load_lib()
    lib.init(local)
    S_full, H = seq_len(w), w["heads"]
    cos, sin = rope_tables(w)
    assert cos.shape == (S_full, 64)
    if ring:
        # Sequence parallel: this rank owns a block of token rows (all heads);
        # K/V chunks go round the ring inside iris_b200_ring_attention().
        assert w["batch"] == 1
        rows_of = np.zeros(world, np.int32)
        a, b = C.c_int(), C.c_int()
        row0 = 0
        for r in range(world):
            lib.iris_b200_seq_shard(S_full, world, r, C.byref(a), C.byref(b))
            rows_of[r] = b.value
            if r == rank:
                row0 = a.value
        S = int(rows_of[rank])
        cos, sin = np.ascontiguousarray(cos[row0:row0 + S]), np.ascontiguousarray(sin[row0:row0 + S])
        entries, h0, nh = [0], 0, H
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = C.create_string_buffer(128)
            assert lib.iris_b200_ring_unique_id(buf) == 0
            ident = torch.tensor(list(buf.raw), dtype=torch.uint8, device="cuda")
        if dist:
            dist.broadcast(ident, src=0)
        assert lib.iris_b200_ring_init(rank, world, bytes(ident.cpu().tolist())) == 0
    else:
        S = S_full
        shard = shard_of(w, rank, world)
        entries, h0, nh = shard if shard else ([], 0, 0)
    width = nh * D                                  # this rank's column slice of every tensor
    d_cos, d_sin = lib.to_device(cos), lib.to_device(sin)
    d_w = lib.to_device(np.ones(D, np.float32))
    scale = 1.0 / np.sqrt(D)

    # Buffer sets: each holds the fused QKV slice of every batch entry this
    # rank owns plus its output; enough sets to exceed L2 (126 MB) several times.
    per_set = len(entries) * S * width * 8
    nsets = max(2, min(8, int(np.ceil(512e6 / max(per_set, 1))))) if entries else 0
    host_qkv = [make_qkv(S, width, 1000 * rank + e) for e in entries]
    sets = []
    for s in range(nsets):
        bufs = []
        for hq in host_qkv:
            dq = lib.alloc(hq.numel() * 2)
            lib.iris_dev_upload(dq, hq.data_ptr(), hq.numel() * 2)
            bufs.append((dq, lib.alloc(S * width * 2)))
        sets.append(bufs)
    lib.check()

    def step(bufs, mark=None):
        for dq, dout in bufs:
            q, k, v = dq, dq + width * 2, dq + 2 * width * 2
            if mark is not None:
                lib.iris_b200_mark(mark + 2)
            lib.iris_b200_qk_norm_rope(q, k, 3 * width, d_w, d_w, d_cos, d_sin, S, nh, D, w["eps"], 0)
            if mark is not None:
                lib.iris_b200_mark(mark)
            if ring:
                rc = lib.iris_b200_ring_attention(dout, width, q, k, v, 3 * width, rows_of.ctypes.data, nh, scale)
                assert rc == 0, rc
            else:
                lib.iris_dev_attention(dout, width, q, k, v, 3 * width, S, S, nh, nh, D, scale, 0, None)
            if mark is not None:
                lib.iris_b200_mark(mark + 1)

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        if entries:
            step(sets[i % nsets])
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = lib.iris_b200_launch_count()
    t_wall0 = time.time()
    lib.iris_b200_mark(0)
    nmark = min(args.steps, 2500)
    for i in range(args.steps):
        if entries:
            step(sets[i % nsets], 2 + 3 * i if (i < nmark and len(entries) == 1) else None)
    lib.iris_b200_mark(1)
    t_enqueued = time.time()
    barrier()
    t_wall1 = time.time()
    ms_total = lib.iris_b200_mark_elapsed_ms(0, 1)
    launches = lib.iris_b200_launch_count() - launches0
    lib.check()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    if dist:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    total_flops = attn_flops(w["batch"], H, S_full, S_full)
    value = total_flops / (ms_step * 1e-3) / 1e12

    # Dominant kernel alone (rank 0): mean launch duration from the marks.
    roof = prologue = None
    bf16_peak, bf16_sust, hbm_peak, src = peaks()
    if rank == 0 and entries and len(entries) == 1:
        durs = [lib.iris_b200_mark_elapsed_ms(2 + 3 * i, 3 + 3 * i) for i in range(min(args.steps, nmark))]
        pdurs = [lib.iris_b200_mark_elapsed_ms(4 + 3 * i, 2 + 3 * i) for i in range(min(args.steps, nmark))]
        pdurs = [d for d in pdurs if d > 0]
        durs = [d for d in durs if d > 0]
        if durs:
            kms = sum(durs) / len(durs)
            achieved = attn_flops(1, nh, S, S_full) / (kms * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": "k_attention_sm100", "achieved": round(achieved, 1),
                    "peak": bf16_peak, "peak_source": src + " bf16 burst", "unit": "TFLOP/s",
                    "frac": round(achieved / bf16_peak, 4), "frac_of_sustained": round(achieved / bf16_sust, 4),
                    "kernel_ms": round(kms, 4), "kernel_ms_median": round(float(np.median(durs)), 4),
                    "kernel_ms_min": round(min(durs), 4), "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(name)}
            if pdurs and not ring:
                pms = sum(pdurs) / len(pdurs)
                pbytes = 4.0 * S * nh * D * 2 + 2.0 * S * 64 * 4     # Q and K read + written, cos + sin read
                prologue = {"bound": "hbm", "kernel": "k_head_norm_rope_128_tok", "achieved": round(pbytes / pms / 1e6, 1),
                            "peak": hbm_peak, "peak_source": src + " HBM copy", "unit": "GB/s",
                            "frac": round(pbytes / pms / 1e6 / hbm_peak, 4), "kernel_ms": round(pms, 4),
                            "kernel_ms_median": round(float(np.median(pdurs)), 4),
                            "kernel_ms_min": round(min(pdurs), 4), "bytes": pbytes}

    # End to end through the C-ABI with host buffers: every step uploads its
    # inputs from pinned memory, runs prologue + attention and downloads the
    # result. Serial: the reference's own blocking upload / download calls.
    # Pipelined (the reported value): the same operations on the library's
    # stream, the copies on two copy streams ordered by events over three
    # device buffer sets, so the upload of step i + 1 and the download of step
    # i - 1 run under the compute of step i.
    e2e = None
    if entries and not args.no_e2e:
        nrep = max(1, min(args.steps, 10))
        host_out = torch.empty((S, width), dtype=torch.bfloat16)
        if torch.cuda.is_available():
            host_out = host_out.pin_memory()
        barrier()
        t0 = time.perf_counter()
        for i in range(nrep):
            bufs = sets[i % nsets]
            for (dq, dout), hq in zip(bufs, host_qkv):
                lib.iris_dev_upload(dq, hq.data_ptr(), hq.numel() * 2)
                lib.iris_dev_upload(d_cos, cos.ctypes.data, cos.nbytes)
                lib.iris_dev_upload(d_sin, sin.ctypes.data, sin.nbytes)
            step(bufs)
            for dq, dout in bufs:
                lib.iris_dev_download(host_out.data_ptr(), dout, S * width * 2)
        torch.cuda.synchronize()
        serial_ms = (time.perf_counter() - t0) * 1e3 / nrep

        nbuf, prep = 3, max(3, min(args.steps, 30))
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        comp = torch.cuda.ExternalStream(int(lib.iris_b200_stream()))
        h_cos, h_sin = torch.from_numpy(cos).pin_memory(), torch.from_numpy(sin).pin_memory()
        dev_in = [[torch.empty((S, 3 * width), dtype=torch.bfloat16, device="cuda") for _ in entries] for _ in range(nbuf)]
        dev_out = [[torch.empty((S, width), dtype=torch.bfloat16, device="cuda") for _ in entries] for _ in range(nbuf)]
        dev_cs = [(torch.empty_like(h_cos, device="cuda"), torch.empty_like(h_sin, device="cuda")) for _ in range(nbuf)]
        pin_out = [[torch.empty((S, width), dtype=torch.bfloat16).pin_memory() for _ in entries] for _ in range(nbuf)]
        ev_up = [torch.cuda.Event() for _ in range(prep)]
        ev_comp = [torch.cuda.Event() for _ in range(prep)]
        ev_down = [torch.cuda.Event() for _ in range(prep)]
        barrier()
        t0 = time.perf_counter()
        for i in range(prep):
            b = i % nbuf
            if i >= nbuf:
                up.wait_event(ev_comp[i - nbuf])          # the last reader of this input set
            with torch.cuda.stream(up):
                for e, hq in enumerate(host_qkv):
                    dev_in[b][e].copy_(hq.view(S, 3 * width), non_blocking=True)
                dev_cs[b][0].copy_(h_cos, non_blocking=True)
                dev_cs[b][1].copy_(h_sin, non_blocking=True)
            ev_up[i].record(up)
            comp.wait_event(ev_up[i])
            if i >= nbuf:
                comp.wait_event(ev_down[i - nbuf])        # the last download of this output set
            for e in range(len(entries)):
                dq, dout = dev_in[b][e].data_ptr(), dev_out[b][e].data_ptr()
                q, k, v = dq, dq + width * 2, dq + 2 * width * 2
                lib.iris_b200_qk_norm_rope(q, k, 3 * width, d_w, d_w, dev_cs[b][0].data_ptr(), dev_cs[b][1].data_ptr(),
                                           S, nh, D, w["eps"], 0)
                if ring:
                    rc = lib.iris_b200_ring_attention(dout, width, q, k, v, 3 * width, rows_of.ctypes.data, nh, scale)
                    assert rc == 0, rc
                else:
                    lib.iris_dev_attention(dout, width, q, k, v, 3 * width, S, S, nh, nh, D, scale, 0, None)
            ev_comp[i].record(comp)
            down.wait_event(ev_comp[i])
            with torch.cuda.stream(down):
                for e in range(len(entries)):
                    pin_out[b][e].copy_(dev_out[b][e], non_blocking=True)
            ev_down[i].record(down)
        torch.cuda.synchronize()
        e_ms = (time.perf_counter() - t0) * 1e3 / prep
        if dist:
            t = torch.tensor([e_ms, serial_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms, serial_ms = float(t[0].item()), float(t[1].item())
        e2e = {"value": round(total_flops / (e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(e_ms, 3),
               "h2d_bytes_per_step": len(entries) * (S * 3 * width * 2 + 2 * cos.nbytes),
               "d2h_bytes_per_step": len(entries) * S * width * 2,
               "how": "copies on two copy streams overlap the neighbouring steps (3 buffer sets)",
               "serial": {"value": round(total_flops / (serial_ms * 1e-3) / 1e12, 2), "ms_per_step": round(serial_ms, 3),
                          "how": "blocking iris_dev_upload / iris_dev_download around every step"}}
    elif dist:
        t = torch.tensor([0.0, 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    lib.check()
    if ring:
        lib.iris_b200_ring_destroy()

    cpu = ref_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_reference(w, budget_s=20.0, steps=1, warmup=0)["cpu_baseline"]
    if rank == 0 and world == 1 and not ring and entries and not args.no_ref_gpu:
        ref_gpu = reference_gpu_kernels(lib, w, sets[0][0], (d_w, d_cos, d_sin), S, nh, scale)

    if rank == 0:
        out = {
            "metric": "joint-attn TFLOP/s per GPU & % bf16 peak at 1/2/4/8 B200 vs host-CPU ref",
            "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": name, "batch": w["batch"], "heads": H, "head_dim": D, "tokens": S_full,
                       "step": "qk_norm_rope + attention", "sharding": "none" if world == 1 and not ring else
                       "ring sequence parallel (K/V rows pushed peer to peer by the copy engines, NCCL for set-up)" if ring else
                       "cfg batch x heads, no collective", "l2": "inputs rotate over %d buffer sets (%.0f MB)" %
                       (nsets, nsets * per_set / 1e6)},
            "per_gpu_tflops": round(value / world, 2),
            "host_enqueue_ms_per_step": round((t_enqueued - t_wall0) * 1e3 / args.steps, 4),
            "pct_bf16_peak": round(100 * value / world / bf16_peak, 2),
            "pct_bf16_sustained": round(100 * value / world / bf16_sust, 2),
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
            "roofline": roof, "roofline_prologue": prologue, "cpu_baseline": cpu, "reference_gpu": ref_gpu,
        }
        print(json.dumps(out))
    if dist:
        dist.destroy_process_group()


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


def cpu_reference(w, budget_s, steps, warmup):
    """Times the reference's CPU code for one step of workload `w` on the host
    cores: Q/K norm + RoPE, then attention. Uses oracle/_ref (the reference
    sources compiled unmodified: BLAS build if it loads, else generic), else
    the CPU port. The sample is a subset of heads sized to the time budget."""
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

    def one(hs):
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
        return time.perf_counter() - t0

    # Head count of the sample. The reference's BLAS build runs one pthread
    # per group of heads (thread count = largest divisor of the head count
    # that fits the cores, fixed at its first call), so samples there are
    # whole multiples of that thread count; its FLUX.3 routine and the
    # generic build walk heads serially. One calibration pass sizes the
    # sample to the time budget, then the timed passes run.
    threads, unit = 1, 1
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
    return {"seconds_per_step": t, "value": val, "heads_sampled": hs,
            "cpu_baseline": {"value": round(val, 5), "unit": "TFLOP/s", "cores": int(threads), "host_cores": ncpu,
                             "kind": kind, "variant": variant,
                             "sample": "%d of %d heads x %d tokens, batch entry 0, fp32, prologue + attention, %.2f s per pass"
                                       % (hs, H, S, t)}}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return
    name = args.workload or ("klein4b-1024" if world == 1 else "klein9b-cfg")
    w = WORKLOADS[name]
    r = cpu_reference(w, budget_s=150.0, steps=args.steps, warmup=args.warmup)
    S = seq_len(w)
    out = {
        "impl": "reference",
        "metric": "joint-attn TFLOP/s per GPU & % bf16 peak at 1/2/4/8 B200 vs host-CPU ref",
        "value": round(r["value"], 5), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(r["seconds_per_step"] * 1e3, 2), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "batch": w["batch"], "heads": w["heads"], "head_dim": D, "tokens": S,
                   "step": "qk_norm + rope + attention on the host CPU"},
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
    ap.add_argument("--mode", default="shard", choices=["shard", "ring"],
                    help="N > 1: independent cfg/head shards (default) or ring sequence parallelism")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip the reference's own CUDA kernels")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
