"""Chunked attention with carried state (split-K over several launches) on one
GPU, and the ring across GPUs when the box has them."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu

D = 128
MAX_ABS, MIN_COS = 2e-2, 0.9999
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.check()


def chunked(lib, q, k, v, H, bounds, mask=None):
    """Attention of q over k/v given as consecutive key chunks [b0, b1), ..."""
    sq, sk = q.shape[0], k.shape[0]
    dq, dk, dv = lib.to_device(q), lib.to_device(k), lib.to_device(v)
    dout = lib.to_device(np.full((sq, H * D), 0x7FC0, np.uint16))
    dstate = lib.alloc(sq * H * D * 4)
    dlse = lib.alloc(sq * H * 4)
    dmask = lib.to_device(np.ascontiguousarray(mask, np.int32)) if mask is not None else None
    for i, (b0, b1) in enumerate(bounds):
        b0, b1 = int(b0), int(b1)
        first, last = i == 0, i == len(bounds) - 1
        rc = lib.iris_b200_attention_chunk(
            dout if last else None, H * D, dq, H * D, dk + b0 * H * D * 2, dv + b0 * H * D * 2, H * D,
            sq, b1 - b0, H, 1.0 / np.sqrt(D), (dmask + b0 * 4) if dmask else None, dstate, dlse,
            int(first), int(last))
        assert rc == 0, rc
    out = ol.from_bf16(lib.to_host(dout, (sq, H * D), np.uint16))
    lib.check()
    for p in (dq, dk, dv, dout, dstate, dlse, dmask):
        if p:
            lib.iris_dev_free(p)
    return out


def check(got, want, H):
    assert np.isfinite(got).all()
    mx, cs = ol.compare_heads(got, want, H)
    assert mx.max() <= MAX_ABS and cs.min() >= MIN_COS, (mx, cs)


def test_split_k_equals_single_pass(lib):
    H, sq, sk = 3, 300, 900
    q, k, v = (ol.to_bf16(ol.randn(40 + i, n, H * D)) for i, n in enumerate((sq, sk, sk)))
    want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), H)
    for bounds in ([(0, 900)], [(0, 130), (130, 387), (387, 451), (451, 900)], [(0, 1), (1, 900)],
                   [(0, 512), (512, 900)]):
        check(chunked(lib, q, k, v, H, bounds), want, H)


def test_split_k_with_mask_and_empty_chunks_of_valid_keys(lib):
    H, sq, sk = 2, 200, 600
    q, k, v = (ol.to_bf16(ol.randn(50 + i, n, H * D)) for i, n in enumerate((sq, sk, sk)))
    mask = np.ones(sk, np.int32)
    mask[:256] = 0                       # the whole first chunk is padding
    mask[500:] = 0
    want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), H, key_mask=mask)
    check(chunked(lib, q, k, v, H, [(0, 256), (256, 430), (430, 600)], mask), want, H)
    none = chunked(lib, q, k, v, H, [(0, 300), (300, 600)], np.zeros(sk, np.int32))
    assert not none.any()


def test_ring_order_emulated_on_one_gpu(lib):
    """Four ranks' worth of work done one after the other: each 'rank' walks
    the chunks in the order the ring would deliver them."""
    H, S, G = 2, 1030, 4
    q, k, v = (ol.to_bf16(ol.randn(60 + i, S, H * D)) for i in range(3))
    want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), H)
    a, b = C.c_int(), C.c_int()
    spans = []
    for r in range(G):
        lib.iris_b200_seq_shard(S, G, r, C.byref(a), C.byref(b))
        spans.append((a.value, a.value + b.value))
    for r in range(G):
        order = [lib.iris_b200_ring_source(r, s, G) for s in range(G)]
        r0, r1 = spans[r]
        # chunks are not contiguous in ring order: gather them
        kk = np.concatenate([k[spans[c][0]:spans[c][1]] for c in order])
        vv = np.concatenate([v[spans[c][0]:spans[c][1]] for c in order])
        edges = np.cumsum([0] + [spans[c][1] - spans[c][0] for c in order])
        got = chunked(lib, np.ascontiguousarray(q[r0:r1]), kk, vv, H, list(zip(edges[:-1], edges[1:])))
        check(got, want[r0:r1], H)


def test_chunk_argument_checks(lib):
    assert lib.iris_b200_attention_chunk(None, 256, 16, 256, 16, 16, 256, 4, 4, 2, 0.1, None, None, None, 1, 0) == 1
    lib.iris_b200_clear_error()
    assert lib.iris_b200_attention_chunk(16, 256, 16, 260, 16, 16, 256, 4, 4, 2, 0.1, None, None, None, 1, 1) == 6
    lib.iris_b200_clear_error()
    # a query stride shorter than a row of heads
    assert lib.iris_b200_attention_chunk(16, 256, 16, 248, 16, 16, 256, 4, 4, 2, 0.1, None, None, None, 1, 1) == 1
    lib.iris_b200_clear_error()


def run_ring_worker(nproc, transport, mode, port, groups=1):
    import torch
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", RING_TEST_TRANSPORT=transport,
               RING_TEST_GROUPS=str(groups))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % nproc,
                          "--master-addr", "127.0.0.1", "--master-port", str(port),
                          os.path.join(ROOT, "tests", "ring_gpu_worker.py"), mode],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "RING_OK" in out.stdout, out.stdout[-3000:]
    if transport == "nccl":
        assert "transport nccl" in out.stdout, out.stdout[-3000:]


@pytest.mark.parametrize("nproc,transport", [(2, "auto"), (2, "nccl"), (4, "auto"), (8, "auto")])
def test_ring_across_gpus(nproc, transport):
    """One process per GPU; `auto` pushes the chunks with the copy engines
    while one attention launch waits for them inside the kernel, `nccl`
    forces the send/recv transport (all chunks first, then the launch)."""
    run_ring_worker(nproc, transport, "toy", 29437)


@pytest.mark.parametrize("nproc,groups,mode", [(4, 2, "toy"), (8, 2, "toy"), (8, 2, "config5"), (8, 4, "toy")])
def test_ring_across_gpus_in_head_groups(nproc, groups, mode):
    """The heads split over independent rings (2 rings of 4 GPUs, 4 rings of
    2, ...): each ring has its own communicator and slot pools, nothing
    crosses between them."""
    run_ring_worker(nproc, "auto", mode, 29441, groups)


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_ring_at_the_multi_reference_shape(nproc):
    """24 heads x 16 896 tokens split over the ranks, sampled rows of every
    rank against the CPU oracle."""
    run_ring_worker(nproc, "auto", "config5", 29439)
