"""Host-side logic of the multi-GPU decompositions, on CPU: shard arithmetic
of the C library, and the ring schedule + state merge run as two gloo ranks
with the CPU oracle standing in for the attention kernel."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle_lib as ol

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    if not os.path.exists(os.path.join(ge.PKG_DIR, "libiris_b200.so")):
        ge.build()
    return ge.load_package().Lib()


def head_shard(lib, heads, n, r):
    a, b = C.c_int(), C.c_int()
    assert lib.iris_b200_head_shard(heads, n, r, C.byref(a), C.byref(b)) == 0
    return a.value, b.value


def test_head_shards_cover_heads_exactly(lib):
    assert [head_shard(lib, 30, 8, r)[1] for r in range(8)] == [4, 4, 4, 4, 4, 4, 3, 3]
    assert [head_shard(lib, 30, 4, r)[1] for r in range(4)] == [8, 8, 7, 7]
    for heads in (24, 30, 32, 7, 1):
        for n in (1, 2, 3, 4, 8, 9):
            spans = [head_shard(lib, heads, n, r) for r in range(n)]
            pos = 0
            for first, count in spans:
                assert first == pos and count >= 0
                pos += count
            assert pos == heads
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    a, b = C.c_int(), C.c_int()
    assert lib.iris_b200_head_shard(24, 4, 4, C.byref(a), C.byref(b)) == 1      # rank out of range
    assert lib.iris_b200_head_shard(24, 0, 0, C.byref(a), C.byref(b)) == 1


def cfg_shard(lib, batch, heads, n, r):
    v = [C.c_int() for _ in range(4)]
    assert lib.iris_b200_cfg_shard(batch, heads, n, r, *[C.byref(x) for x in v]) == 0
    return tuple(x.value for x in v)


def test_cfg_split_assigns_every_entry_head_once(lib):
    # cond / uncond x 32 heads (the 9B base model) over 1, 2, 4, 8 GPUs
    for n in (1, 2, 4, 8, 3, 5):
        seen = np.zeros((2, 32), int)
        for r in range(n):
            e0, es, h0, nh = cfg_shard(lib, 2, 32, n, r)
            for e in range(e0, 2, es):
                seen[e, h0:h0 + nh] += 1
        assert (seen == 1).all(), (n, seen)
    assert cfg_shard(lib, 2, 32, 2, 1) == (1, 2, 0, 32)
    assert cfg_shard(lib, 2, 32, 8, 5) == (1, 2, 8, 8)
    assert cfg_shard(lib, 2, 32, 1, 0) == (0, 1, 0, 32)


def test_ring_schedule_visits_every_chunk_once(lib):
    for n in (1, 2, 4, 8):
        for r in range(n):
            src = [lib.iris_b200_ring_source(r, s, n) for s in range(n)]
            assert sorted(src) == list(range(n)) and src[0] == r
            # what arrives at step s + 1 is what the previous rank held at step s
            for s in range(n - 1):
                assert src[s + 1] == lib.iris_b200_ring_source((r - 1) % n, s, n)
    assert lib.iris_b200_ring_source(0, 0, 0) == -1
    a, b = C.c_int(), C.c_int()
    assert lib.iris_b200_seq_shard(16896, 8, 3, C.byref(a), C.byref(b)) == 0 and (a.value, b.value) == (6336, 2112)


def ring_plan(lib, n, max_parts=0):
    first, count = (C.c_int * max(n, 1))(), (C.c_int * max(n, 1))()
    nl = lib.iris_b200_ring_plan(n, max_parts, first, count)
    return [(first[i], count[i]) for i in range(max(nl, 0))], nl


def test_ring_plan_covers_the_steps_in_order(lib):
    for n in range(1, 17):
        for max_parts in (0, 1, 2, 3, 8):
            plan, nl = ring_plan(lib, n, max_parts)
            assert nl == len(plan) >= 1
            steps = [s for f, c in plan for s in range(f, f + c)]
            assert steps == list(range(n))                       # every step once, in arrival order
            assert all(c >= 1 for _, c in plan)
            sizes = [c for _, c in plan]
            if max_parts:
                assert nl == min(n, max_parts) and max(sizes) - min(sizes) <= 1      # as even as they come
            else:
                assert nl == min(n, 4)
                assert nl == 1 or sizes[-1] == 1                 # what arrives last is a part of its own
                assert sizes[:-1] == sorted(sizes[:-1], reverse=True) and max(sizes[:-1] or [1]) - min(sizes[:-1] or [1]) <= 1
    assert ring_plan(lib, 8)[0] == [(0, 3), (3, 2), (5, 2), (7, 1)]
    assert ring_plan(lib, 8, 4)[0] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert ring_plan(lib, 4)[0] == [(0, 1), (1, 1), (2, 1), (3, 1)]
    assert ring_plan(lib, 2)[0] == [(0, 1), (1, 1)]
    assert ring_plan(lib, 7, 2)[0] == [(0, 3), (3, 4)]
    assert lib.iris_b200_ring_plan(0, 1, None, None) == -1


def test_grouped_steps_merge_like_single_steps(lib):
    """The merge of partial results does not care how the keys are grouped:
    eight chunks merged one by one and by the 8-rank plan agree."""
    H, D, S, n = 2, 128, 64, 8
    q, k, v = (ol.randn(30 + i, S * n if i else S, H * D) for i in range(3))
    scale = 1 / np.sqrt(D)

    def run(groups):
        out = np.zeros((S, H, D), np.float32)
        lse = np.full((S, H), -np.inf, np.float32)
        for f, c in groups:
            kc, vc = k[f * S:(f + c) * S], v[f * S:(f + c) * S]
            o_c = ol.dev_attention(q, kc, vc, H).reshape(S, H, D)
            sc = np.einsum("qhd,khd->hqk", q.reshape(S, H, D), kc.reshape(-1, H, D)) * scale * np.log2(np.e)
            lse_c = (np.log2(np.exp2(sc - sc.max(2, keepdims=True)).sum(2)) + sc.max(2)).T
            new = np.logaddexp2(lse, lse_c)
            out = out * np.exp2(lse - new)[:, :, None] + o_c * np.exp2(lse_c - new)[:, :, None]
            lse = new
        return out.reshape(S, H * D)

    want = ol.dev_attention(q, k, v, H)
    single = run([(s, 1) for s in range(n)])
    grouped = run(ring_plan(lib, n)[0])
    assert np.abs(single - want).max() < 2e-5 and np.abs(grouped - want).max() < 2e-5


WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, ROOT)
import oracle_lib as ol
import __graft_entry__ as ge
lib = ge.load_package().Lib()
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
H, D, S = 2, 128, 150                       # 150 rows: uneven 75 / 75, 3 ranks would be 50 each
import ctypes as C
a, b = C.c_int(), C.c_int()
rows_of = []
for r in range(world):
    lib.iris_b200_seq_shard(S, world, r, C.byref(a), C.byref(b)); rows_of.append((a.value, b.value))
q, k, v = (ol.randn(10 + i, S, H * D) for i in range(3))
r0, n = rows_of[rank]
ql = q[r0:r0 + n]
chunk = np.concatenate([k[r0:r0 + n], v[r0:r0 + n]], 1)
out = np.zeros((n, H * D), np.float32); lse = np.full((n, H), -np.inf, np.float32)
scale = 1 / np.sqrt(D)
for s in range(world):
    src = lib.iris_b200_ring_source(rank, s, world)
    assert chunk.shape[0] == rows_of[src][1]
    if s + 1 < world:                        # forward the resident chunk, receive the next
        nxt_src = lib.iris_b200_ring_source(rank, s + 1, world)
        recv = torch.empty((rows_of[nxt_src][1], 2 * H * D))
        ops = [dist.P2POp(dist.isend, torch.from_numpy(chunk.copy()), (rank + 1) % world),
               dist.P2POp(dist.irecv, recv, (rank - 1) % world)]
        reqs = dist.batch_isend_irecv(ops)
    kc, vc = chunk[:, :H * D], chunk[:, H * D:]
    # chunk attention on the CPU oracle + its log2-sum-exp, merged like the kernel does
    o_c = ol.dev_attention(ql, kc, vc, H)
    sc = np.einsum("qhd,khd->hqk", ql.reshape(n, H, D), kc.reshape(-1, H, D)) * scale * np.log2(np.e)
    lse_c = np.log2(np.exp2(sc - sc.max(2, keepdims=True)).sum(2)) + sc.max(2)          # [H, n]
    lse_c = lse_c.T
    new = np.logaddexp2(lse, lse_c)
    wp, wc = np.exp2(lse - new), np.exp2(lse_c - new)
    out = (out.reshape(n, H, D) * wp[:, :, None] + o_c.reshape(n, H, D) * wc[:, :, None]).reshape(n, H * D)
    lse = new
    if s + 1 < world:
        for rq in reqs: rq.wait()
        chunk = recv.numpy().copy()
want = ol.dev_attention(q, k, v, H)[r0:r0 + n]
err = float(np.abs(out - want).max())
res = torch.tensor([err]); dist.all_reduce(res, op=dist.ReduceOp.MAX)
if rank == 0: print("RING_MAX_ERR %.3e" % res.item())
dist.destroy_process_group()
'''


def test_ring_schedule_and_merge_on_two_gloo_ranks(lib, tmp_path):
    script = tmp_path / "ring_worker.py"
    script.write_text("ROOT = %r\n" % ROOT + WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29431", str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stdout + out.stderr
    line = [l for l in out.stdout.splitlines() if l.startswith("RING_MAX_ERR")][0]
    assert float(line.split()[1]) < 2e-5


# ---------------------------------------------------------------------------
# how a launch cuts its keys (pure host arithmetic, no device)
# ---------------------------------------------------------------------------

def runs_plan(pkg, lib, runs, seq_q, heads, nparts, sms=148):
    arr = (pkg.binding.KeyRun * len(runs))()
    for i, r in enumerate(runs):
        arr[i].view, arr[i].row0, arr[i].rows, arr[i].arrive = r[:4]
        arr[i].rows_per_word = r[4] if len(r) > 4 else 0
    tiles = (C.c_int * 9)()
    nkv = C.c_int()
    n = lib.iris_b200_attention_runs_plan(arr, len(runs), seq_q, heads, nparts, sms, tiles, C.byref(nkv))
    return n, list(tiles[:max(n, 0) + 1]), nkv.value


def test_key_parts_of_a_launch(lib):
    import __graft_entry__ as ge
    pkg = ge.load_package()
    # one run, library's choice: the headline shape fills the SMs without a split, the 768-token one is cut in two
    assert runs_plan(pkg, lib, [(0, 0, 4608, -1)], 4608, 24, 0) == (1, [0, 36], 36)
    assert runs_plan(pkg, lib, [(0, 0, 768, -1)], 768, 24, 0) == (2, [0, 3, 6], 6)
    # one rank's share of the 8-rank ring as a plain launch: two parts of equal tiles
    n, tiles, nkv = runs_plan(pkg, lib, [(0, 0, 16896, -1)], 2112, 24, 0)
    assert (n, tiles, nkv) == (2, [0, 66, 132], 132)
    # ragged runs: every run ends in a partial tile of its own; forced parts fall on run boundaries
    runs = [(0, 5, 130, -1), (1, 11, 257, -1), (0, 140, 64, -1), (1, 279, 1, -1), (0, 209, 511, -1)]
    n, tiles, nkv = runs_plan(pkg, lib, runs, 300, 3, 3)
    assert nkv == 2 + 3 + 1 + 1 + 4 and n == 3
    starts = [0, 2, 5, 6, 7, 11]                                  # first tile of every run, and the end
    assert tiles[0] == 0 and tiles[-1] == nkv and all(t in starts for t in tiles)
    assert tiles == sorted(set(tiles))                            # no empty part
    # more parts than runs: as many as there are runs
    assert runs_plan(pkg, lib, runs[:2], 300, 3, 8)[0] == 2
    assert runs_plan(pkg, lib, runs, 300, 3, 1) == (1, [0, nkv], nkv)
    # bad arguments
    assert runs_plan(pkg, lib, [(2, 0, 10, -1)], 10, 1, 0)[0] == -1
    assert runs_plan(pkg, lib, [(0, 0, 0, -1)], 10, 1, 0)[0] == -1


@pytest.mark.parametrize("G", [1, 2, 3, 4, 8, 16])
def test_ring_launch_plan(lib, G):
    """The attention launch of every rank of a ring call: runs in ring order,
    slots guarded by their arrival words, parts on the step boundaries of
    iris_b200_ring_plan (moved down to a tile boundary), never empty."""
    import __graft_entry__ as ge
    pkg = ge.load_package()
    for S in (16896, 2037, 4608):
        a, b = C.c_int(), C.c_int()
        rows_of = []
        for r in range(G):
            lib.iris_b200_seq_shard(S, G, r, C.byref(a), C.byref(b))
            rows_of.append(b.value)
        rows = np.array(rows_of, np.int32)
        even = len(set(rows_of)) == 1
        for rank in range(G):
            runs = (pkg.binding.KeyRun * 16)()
            tiles = (C.c_int * 9)()
            nkv = C.c_int()
            code = lib.iris_b200_ring_launch_plan(rank, G, rows.ctypes.data, 24, 0, 148, runs, tiles, C.byref(nkv))
            assert code > 0
            nruns, nparts = divmod(code, 100)
            assert (runs[0].view, runs[0].row0, runs[0].rows, runs[0].arrive) == (0, 0, rows_of[rank], -1)
            if G == 1:
                assert nruns == 1
                continue
            plan, npl = ring_plan(lib, G)
            assert nparts == npl
            if even:
                assert nruns == 2 and runs[1].rows == (G - 1) * rows_of[rank] and runs[1].rows_per_word == rows_of[rank]
                assert runs[1].arrive == 1 and runs[1].row0 == rows_of[rank]
                total_tiles = -(-rows_of[rank] // 128) + -(-(G - 1) * rows_of[rank] // 128)
            else:
                assert nruns == G
                slot = max(rows_of)
                for s in range(1, G):
                    src = lib.iris_b200_ring_source(rank, s, G)
                    assert (runs[s].view, runs[s].row0, runs[s].rows, runs[s].arrive) == (1, s * slot, rows_of[src], s)
                total_tiles = sum(-(-runs[i].rows // 128) for i in range(nruns))
            assert nkv.value == total_tiles
            t = list(tiles[:nparts + 1])
            assert t[0] == 0 and t[-1] == total_tiles and t == sorted(set(t))
            # a part never starts before the rows of its first step begin
            first_row = np.concatenate([[0], np.cumsum([rows_of[lib.iris_b200_ring_source(rank, s, G)] for s in range(G)])])
            for i, (f, _) in enumerate(plan):
                if even or f == 0:
                    own_tiles = -(-rows_of[rank] // 128)
                    want = 0 if f == 0 else own_tiles + (int(first_row[f]) - rows_of[rank]) // 128
                    assert t[i] == want


@pytest.mark.parametrize("world,heads_per_ring", [(4, 12), (8, 6)])
def test_launch_plan_of_rings_of_two(lib, world, heads_per_ring):
    """Head groups x rings of two over the 16 896-token sequence (what the
    bench runs from four GPUs up): when the one chunk is expected in time the
    ring call asks for one part, and the launch's own cost model then cuts the
    keys where it pays. At eight GPUs (198 query blocks on 148 SMs) that is
    two parts whose boundary is the partner's slot: own rows first."""
    import __graft_entry__ as ge
    pkg = ge.load_package()
    a, b = C.c_int(), C.c_int()
    rows_of = []
    for r in range(2):
        lib.iris_b200_seq_shard(16896, 2, r, C.byref(a), C.byref(b))
        rows_of.append(b.value)
    assert rows_of == [8448, 8448]
    rows = np.array(rows_of, np.int32)
    for rank in range(2):
        runs = (pkg.binding.KeyRun * 16)()
        tiles = (C.c_int * 9)()
        nkv = C.c_int()
        code = lib.iris_b200_ring_launch_plan(rank, 2, rows.ctypes.data, heads_per_ring, 1, 148, runs, tiles, C.byref(nkv))
        nruns, nparts = divmod(code, 100)
        assert nruns == 2 and nkv.value == 132
        assert (runs[1].view, runs[1].row0, runs[1].rows, runs[1].arrive) == (1, 8448, 8448, 1)
        if world == 8:
            assert nparts == 2 and list(tiles[:3]) == [0, 66, 132]
        else:
            assert nparts == 1 and list(tiles[:2]) == [0, 132]      # 396 blocks: three full rounds, no cut


# ---------------------------------------------------------------------------
# work list of a linear-layer launch (host arithmetic shared with the launcher)
# ---------------------------------------------------------------------------

def linear_plan(lib, rows, split, cin, out, glu_cols, sms=148):
    tm, tn, band = C.c_int(), C.c_int(), C.c_int()
    n = lib.iris_b200_linear_plan(rows, split, cin, out, glu_cols, sms, C.byref(tm), C.byref(tn), C.byref(band), None, 0)
    assert n == tm.value * tn.value
    order = np.zeros((n, 4), np.int32)
    assert lib.iris_b200_linear_plan(rows, split, cin, out, glu_cols, sms, C.byref(tm), C.byref(tn), C.byref(band),
                                     order.ctypes.data, n) == n
    return tm.value, tn.value, band.value, order


@pytest.mark.parametrize("rows,split,cin,out,glu", [(4608, 4608, 3072, 9216, 9216), (4608, 512, 3072, 9216, 0),
                                                    (4608, 4608, 12288, 3072, 0), (4608, 512, 9216, 3072, 0),
                                                    (300, 77, 256, 0, 200), (129, 0, 64, 264, 0), (5, 5, 64, 8, 0)])
def test_linear_work_list_covers_every_tile_once(lib, rows, split, cin, out, glu):
    tm, tn, band, order = linear_plan(lib, rows, split, cin, out, glu)
    assert tm == -(-split // 128) + -(-(rows - split) // 128)
    assert tn == -(-out // 256) + -(-glu // 128)
    assert 1 <= band <= max(tn, 1)
    seen = set()
    for m0, row_end, nt, is_glu in order:
        assert (m0, nt) not in seen
        seen.add((int(m0), int(nt)))
        # a row tile stays inside its row group
        assert (m0 < split and row_end == split) or (m0 >= split and row_end == rows)
        assert m0 < row_end and (m0 - (0 if m0 < split else split)) % 128 == 0
        assert bool(is_glu) == (nt >= -(-out // 256))
    assert len(seen) == tm * tn
    # every row is covered by exactly one row tile
    firsts = sorted({m for m, _ in seen})
    covered = sum(min(128, (split if m < split else rows) - m) for m in firsts)
    assert covered == rows


def test_linear_work_list_order_follows_the_l2_working_set(lib):
    """Small x (the input projections): all row tiles of a column tile are
    adjacent. Large x and long rows (the output projection of a single block:
    113 MB of activations, 75 MB of weights): all column tiles of a row tile
    are adjacent, so that the ~148 tiles in flight share 12 row tiles."""
    _, tn, band, order = linear_plan(lib, 4608, 4608, 3072, 9216, 9216)
    assert band == 1 and (order[:36, 2] == 0).all() and len(set(order[:36, 0])) == 36
    _, tn, band, order = linear_plan(lib, 4608, 4608, 12288, 3072, 0)
    assert band == tn == 12 and (order[:12, 0] == 0).all() and sorted(order[:12, 2]) == list(range(12))
    assert lib.iris_b200_linear_plan(10, 11, 64, 8, 0, 148, None, None, None, None, 0) == -1


# ---------------------------------------------------------------------------
# what bench.py gives every rank of a multi-GPU run (host arithmetic only)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("world,groups", [(2, 1), (4, 2), (8, 4), (8, 2), (8, 1)])
def test_bench_head_groups_and_rings_cover_the_workload_once(lib, world, groups):
    """Head groups x rings over the 16 896-token workload: the ranks of a ring
    hold disjoint row blocks that tile the sequence, the rings hold disjoint
    head groups that tile the heads, and every (row, head) belongs to exactly
    one rank."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench

    class Rank:
        pass

    w = bench.WORKLOADS["flux3-multiref"]
    S, H = bench.seq_len(w), w["heads"]
    owner = np.zeros((S, H), np.int32)
    size = world // groups
    for rank in range(world):
        job = Rank()
        job.lib, job.rank, job.world = lib, rank, world
        p = bench.plan_of(job, w, "ring", groups)
        assert p["S"] == int(p["rows_of"][rank % size]) and len(p["rows_of"]) == size
        assert int(np.sum(p["rows_of"])) == S and p["row0"] == int(np.sum(p["rows_of"][:rank % size]))
        assert p["nh"] == H // groups and p["h0"] == (rank // size) * (H // groups)
        owner[p["row0"]:p["row0"] + p["S"], p["h0"]:p["h0"] + p["nh"]] += 1
    assert (owner == 1).all()
