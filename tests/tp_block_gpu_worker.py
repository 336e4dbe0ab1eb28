"""One rank of the tensor-parallel block test (launched by test_gpu_block_tp.py
through torch.distributed.run): heads and MLP columns sharded over the ranks,
hidden-state rows owned by the ranks, two blocks in a row (the two sets of the
staging buffers), result gathered and checked against the CPU restatement of
the unsharded block."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import block_cases as bc         # noqa: E402
import __graft_entry__ as ge     # noqa: E402

D = 128


def shard_weights(inp, r, G):
    H, mlp, dim = inp["heads"], inp["mlp"], inp["dim"]
    hl, ml = H // G, mlp // G
    hs, ms = slice(r * hl * D, (r + 1) * hl * D), slice(r * ml, (r + 1) * ml)
    w_in, w_out = inp["w_in"], inp["w_out"]
    q, k, v = w_in[:dim], w_in[dim:2 * dim], w_in[2 * dim:3 * dim]
    gate, up = w_in[3 * dim:3 * dim + mlp], w_in[3 * dim + mlp:]
    win = np.ascontiguousarray(np.concatenate([q[hs], k[hs], v[hs], gate[ms], up[ms]], 0))
    wout = np.ascontiguousarray(np.concatenate([w_out[:, :dim][:, hs], w_out[:, dim:][:, ms]], 1))
    return win, wout, hl, ml


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = ge.load_package().load()
    lib.init(int(os.environ.get("LOCAL_RANK", rank)))
    ident = [bytes(128)]
    if rank == 0:
        buf = C.create_string_buffer(128)
        assert lib.iris_b200_ring_unique_id(buf) == 0
        ident = [buf.raw]
    dist.broadcast_object_list(ident, src=0)
    assert lib.iris_b200_ring_init(rank, world, ident[0]) == 0
    worst = torch.tensor([0.0, -1.0])
    base = dict(bc.MID, heads=2 * world, mlp=384 * world)
    cases = [dict(base, name="tp-even", txt=64, img=(8, 3 * world * 4)), dict(base, name="tp-uneven", txt=40, img=(12, 11)),
             # an odd number of heads per rank: the Q | K | V columns end in the middle of a 256-column tile
             dict(base, name="tp-odd-heads", heads=3 * world, mlp=392 * world, txt=40, img=(12, 11))]
    if len(sys.argv) > 1 and sys.argv[1] == "klein4b":
        cases = [dict(bc.KLEIN4B_SHORT, name="tp-klein4b", txt=128, img=(16, 24))]
    for case in cases:
        inp = bc.block_inputs(case)
        seq, dim = inp["seq"], inp["dim"]
        a, b = C.c_int(), C.c_int()
        rows = []
        for r in range(world):
            lib.iris_b200_seq_shard(seq, world, r, C.byref(a), C.byref(b))
            rows.append((a.value, b.value))
        rows_of = np.array([n for _, n in rows], np.int32)
        r0, n = rows[rank]
        win, wout, hl, ml = shard_weights(inp, rank, world)
        dx = lib.to_device(np.ascontiguousarray(inp["x"][r0:r0 + n]))
        ptrs = [lib.to_device(t) for t in (win, wout, inp["norm_q"], inp["norm_k"], inp["mod"], inp["cos"], inp["sin"])]
        scratch = lib.alloc(lib.iris_b200_single_block_tp_scratch_bytes(seq, hl, ml))
        calls = 3
        # The waits inside the kernels are bounded (1 s by default): the ranks have to enter a block within that
        # time of one another, and rank 0 has just spent seconds in the CPU restatement of the previous case.
        dist.barrier()
        for _ in range(calls):
            rc = lib.iris_b200_single_block_tp(dx, scratch, *ptrs, rows_of.ctypes.data, dim, hl, ml, None)
            assert rc == 0, rc
        mine = lib.to_host(dx, (n, dim), np.float32)
        lib.check()
        for p in [dx, scratch] + ptrs:
            lib.iris_dev_free(p)
        parts = [None] * world
        dist.all_gather_object(parts, mine)
        if rank == 0:
            got = np.concatenate(parts, 0)
            want = inp["x"]
            for _ in range(calls):
                want = bc.oracle_block(dict(inp, x=want))
            rel, cos = bc.delta_metrics(got, want, inp["x"])
            assert np.isfinite(got).all()
            worst = torch.maximum(worst, torch.tensor([float(rel), -float(cos)]))
    lib.iris_b200_ring_destroy()
    if rank == 0:
        ok = worst[0].item() <= 2e-2 and -worst[1].item() >= 0.9999
        print("TP_%s rel %.4g cos %.6f" % ("OK" if ok else "FAIL", worst[0].item(), -worst[1].item()))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
