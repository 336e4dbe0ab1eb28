"""One rank of the row-parallel out-projection test (launched by
test_gpu_outproj.py through torch.distributed.run, or run alone as a group of
one): x_rows += gate * (cat . W^T)[own rows], with the reduction over the
ranks' column slices done by the GEMM epilogue over NVLink; checked against a
float64 product of the same bf16 operands."""
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
    ident = [bytes(128)]
    if rank == 0:
        buf = C.create_string_buffer(128)
        assert lib.iris_b200_ring_unique_id(buf) == 0
        ident = [buf.raw]
    dist.broadcast_object_list(ident, src=0)
    assert lib.iris_b200_ring_init(rank, world, ident[0]) == 0
    worst = 0.0
    # (seq, heads, gate?) : even rows; uneven rows and heads with a ragged last tile; larger staging (pool grows)
    for case, (S, H, use_gate) in enumerate(((256 * world, 2 * world, True), (700, 3 * world + 1, False),
                                             (1500, 4 * world, True))):
        for rep in range(3):                     # consecutive calls alternate between the two staging sets
            worst = max(worst, one_case(lib, rank, world, S, H, use_gate, 100 * case + rep))
    t = torch.tensor([worst])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    lib.check()
    lib.iris_b200_ring_destroy()
    if rank == 0:
        print("OUTPROJ_%s max_rel_err %.3g" % ("OK" if t.item() <= 2e-3 else "FAIL", t.item()))
    dist.destroy_process_group()


def one_case(lib, rank, world, S, H, use_gate, seed):
    dim = H * D
    cat = ol.to_bf16(ol.randn(300 + seed, S, dim))
    W = ol.to_bf16(ol.randn(301 + seed, dim, dim) / np.sqrt(dim))
    x = ol.randn(302 + seed, S, dim)
    gate = ol.randn(303 + seed, 1, dim)[0] if use_gate else None
    a, b = C.c_int(), C.c_int()
    rows_of, spans, heads_of = [], [], []
    for r in range(world):
        lib.iris_b200_seq_shard(S, world, r, C.byref(a), C.byref(b))
        rows_of.append(b.value)
        spans.append((a.value, a.value + b.value))
        lib.iris_b200_head_shard(H, world, r, C.byref(a), C.byref(b))
        heads_of.append((a.value, b.value))
    rows_of = np.array(rows_of, np.int32)
    h0, nh = heads_of[rank]
    k0, k = h0 * D, nh * D
    r0, r1 = spans[rank]
    d_cat = lib.to_device(np.ascontiguousarray(cat[:, k0:k0 + k]))       # this rank's head columns, all rows
    d_W = lib.to_device(W)                                               # the full matrix; the rank reads its column slice
    d_x = lib.to_device(np.ascontiguousarray(x[r0:r1]))
    d_gate = lib.to_device(gate) if use_gate else None
    rc = lib.iris_b200_outproj_residual(d_x, d_cat, k, d_W + k0 * 2, dim, d_gate, rows_of.ctypes.data, k, dim)
    assert rc == 0, rc
    got = lib.to_host(d_x, (r1 - r0, dim), np.float32)
    lib.check()
    for p in (d_cat, d_W, d_x, d_gate):
        if p:
            lib.iris_dev_free(p)
    prod = ol.from_bf16(cat[r0:r1]).astype(np.float64) @ ol.from_bf16(W).astype(np.float64).T
    want = x[r0:r1] + (gate[None, :] if use_gate else 1.0) * prod
    assert np.isfinite(got).all()
    return float(np.abs(got - want).max() / max(1.0, np.abs(want).max()))


if __name__ == "__main__":
    main()
