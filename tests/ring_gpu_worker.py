"""One rank of the multi-GPU ring test (launched by test_gpu_chunks.py through
torch.distributed.run): local rows through the ring attention, result
checked against the CPU oracle over the full sequence.

    ring_gpu_worker.py toy       small shapes, even and uneven rows, all rows checked
    ring_gpu_worker.py config5   24 heads x 16 896 tokens (the FLUX.3 multi-reference
                                 shape), sampled query rows of every rank checked

RING_TEST_TRANSPORT=nccl selects the send/recv transport. RING_TEST_GROUPS=g
splits the heads over g independent rings of world / g ranks each (ranks
[i * world / g, (i + 1) * world / g) form ring i and take head slice i)."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle_lib as ol          # noqa: E402
import __graft_entry__ as ge     # noqa: E402

D = 128


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = ge.load_package().load()
    lib.init(int(os.environ.get("LOCAL_RANK", rank)))
    groups = int(os.environ.get("RING_TEST_GROUPS", "1"))
    assert world % groups == 0
    size = world // groups
    grp, rr = rank // size, rank % size
    mine = None
    if rr == 0:                                # the first rank of every ring makes its id
        buf = C.create_string_buffer(128)
        assert lib.iris_b200_ring_unique_id(buf) == 0
        mine = buf.raw
    ids = [None] * world
    dist.all_gather_object(ids, mine)
    nccl = os.environ.get("RING_TEST_TRANSPORT", "auto") == "nccl"
    assert lib.iris_b200_ring_configure(1 if nccl else 0, 0) == 0
    assert lib.iris_b200_ring_init(rr, size, ids[grp * size]) == 0

    worst = torch.tensor([0.0, -1.0])
    mode = sys.argv[1] if len(sys.argv) > 1 else "toy"
    if mode == "config5":
        cases = ((24 // groups, 16896, 24),)
    else:
        # equal rows per rank (the slots then form one run of rows), a length that leaves
        # a partial tile in every slot, then uneven rows, which also makes the pool grow
        cases = ((2, 384 * size, None), (3, 200 * size, None), (4, 2000 + 37, None))
    for H, S, nsample in cases:               # H heads per ring
        res = one_case(lib, rr, size, H, S, nsample, grp, groups)
        worst = torch.maximum(worst, res)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    transport = lib.iris_b200_ring_transport()
    lib.iris_b200_ring_destroy()
    if rank == 0:
        ok = worst[0].item() <= 2e-2 and -worst[1].item() >= 0.9999
        print("RING_%s max_abs %.4g min_cos %.6f transport %s" % (
            "OK" if ok else "FAIL", worst[0].item(), -worst[1].item(), "nccl" if transport == 1 else "copy-engine"))
    dist.destroy_process_group()


def one_case(lib, rank, world, H, S, nsample, grp=0, groups=1):
    """rank / world: this rank inside its ring. The ring takes heads
    [grp * H, (grp + 1) * H) of tensors generated for groups * H heads."""
    cols = slice(grp * H * D, (grp + 1) * H * D)
    q, k, v = (np.ascontiguousarray(ol.to_bf16(ol.randn(70 + i, S, groups * H * D))[:, cols]) for i in range(3))
    a, b = C.c_int(), C.c_int()
    rows = []
    for r in range(world):
        lib.iris_b200_seq_shard(S, world, r, C.byref(a), C.byref(b))
        rows.append((a.value, b.value))
    rows_of = np.array([n for _, n in rows], np.int32)
    r0, n = rows[rank]
    fused = np.ascontiguousarray(np.concatenate([q[r0:r0 + n], k[r0:r0 + n], v[r0:r0 + n]], 1))
    dqkv = lib.to_device(fused)
    dout = lib.alloc(n * H * D * 2)
    w = H * D * 2
    for rep in range(3):                      # repeated calls reuse buffers and communicator
        rc = lib.iris_b200_ring_attention(dout, H * D, dqkv, dqkv + w, dqkv + 2 * w, 3 * H * D,
                                          rows_of.ctypes.data, H, 1.0 / np.sqrt(D))
        assert rc == 0, rc
    got = ol.from_bf16(lib.to_host(dout, (n, H * D), np.uint16))
    lib.check()
    for p in (dqkv, dout):
        lib.iris_dev_free(p)
    if nsample is None:
        rows = np.arange(r0, r0 + n, dtype=np.int32)
    else:                                     # the block's edges and a seeded sample in between
        rng = np.random.default_rng(11 + rank)
        rows = np.unique(np.concatenate([[r0, r0 + 127, r0 + 128, r0 + n - 1], r0 + rng.integers(0, n, nsample)]))
        rows = rows.astype(np.int32)
    want = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), H, rows=rows)
    mx, cs = ol.compare_heads(got[rows - r0], want[rows], H)
    assert np.isfinite(got).all()
    return torch.tensor([float(mx.max()), -float(cs.min())])


if __name__ == "__main__":
    main()
