"""The ring protocol on host threads (iris_b200_ring_loopback): known-answer
runs and the failure paths, with every fault injected on the host. Runs
without a GPU."""
import ctypes as C

import numpy as np
import pytest

OK, ETIMEOUT, EPROTO = 0, 3, 8
DROP, DELAY, CORRUPT, LEAVE, BAD_ROWS = 1, 2, 3, 4, 5


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="module")
def lib(pkg):
    return pkg.Lib()


def loopback(pkg, lib, rows_of, calls=4, row_bytes=96, wait_us=400000, faults=()):
    G = len(rows_of)
    rows = np.array(rows_of, np.int32)
    arr = (pkg.binding.LoopFault * max(len(faults), 1))()
    for i, f in enumerate(faults):
        arr[i].kind, arr[i].rank, arr[i].call, arr[i].step = f[:4]
        arr[i].delay_us = f[4] if len(f) > 4 else 0
    status, done = np.full(G, -1, np.int32), np.full(G, -1, np.int32)
    digest = np.zeros(G, np.uint64)
    rc = lib.iris_b200_ring_loopback(G, rows.ctypes.data, row_bytes, calls, wait_us, arr, len(faults),
                                     status.ctypes.data, digest.ctypes.data, done.ctypes.data)
    assert rc == 0
    want = [lib.iris_b200_ring_loopback_digest(G, rows.ctypes.data, row_bytes, calls, r) for r in range(G)]
    return status, digest, done, np.array(want, np.uint64)


@pytest.mark.parametrize("rows_of", [[5], [7, 7], [33, 31, 32], [16] * 8, [9, 1, 30, 2, 17, 17, 3, 11], [4] * 16])
def test_fault_free_runs_have_the_known_answer(pkg, lib, rows_of):
    """Many calls back to back over two pool sets and no acknowledgements:
    every chunk of every call arrives intact (a chunk overwritten too early
    would fail its checksum) and the digests are the sequentially computed
    ones."""
    status, digest, done, want = loopback(pkg, lib, rows_of, calls=12)
    assert (status == OK).all() and (done == 12).all()
    assert (digest == want).all()


def test_a_dropped_chunk_times_out_its_consumer_and_nobody_blocks(pkg, lib):
    status, _, done, _ = loopback(pkg, lib, [8] * 4, calls=5, wait_us=50000, faults=[(DROP, 1, 3, 2)])
    # rank 1 + 2 steps = rank 3 never gets call 3: its wait runs out, or, when rank 1's push of call 4
    # overtakes the limit, the arrival word moves on and the slot still holds the rows of call 1
    assert status[3] in (ETIMEOUT, EPROTO) and done[3] == 2
    # the others complete call 3; call 4 needs rank 3, which is gone, so they time out there
    for r in (0, 1, 2):
        assert status[r] == ETIMEOUT and done[r] == 3


def test_a_delayed_chunk_is_waited_for(pkg, lib):
    status, digest, done, want = loopback(pkg, lib, [8, 9, 10], calls=4, wait_us=400000,
                                          faults=[(DELAY, 2, 2, 1, 30000)])
    assert (status == OK).all() and (digest == want).all() and (done == 4).all()


def test_a_delay_beyond_the_limit_is_a_timeout(pkg, lib):
    status, _, _, _ = loopback(pkg, lib, [8, 8], calls=2, wait_us=5000, faults=[(DELAY, 0, 1, 1, 100000)])
    assert status[1] == ETIMEOUT


def test_a_corrupted_chunk_is_a_protocol_error(pkg, lib):
    status, _, done, _ = loopback(pkg, lib, [12] * 4, calls=3, wait_us=50000, faults=[(CORRUPT, 2, 2, 3)])
    assert status[1] == EPROTO and done[1] == 1           # rank 2 + 3 steps = rank 1
    assert all(s in (ETIMEOUT, OK) for i, s in enumerate(status) if i != 1)


def test_ranks_that_disagree_about_a_row_count(pkg, lib):
    status, _, _, _ = loopback(pkg, lib, [6, 7, 8], calls=2, wait_us=50000, faults=[(BAD_ROWS, 0, 1, -1)])
    assert status[1] == EPROTO and status[2] == EPROTO    # both consumers of rank 0's rows
    assert status[0] in (OK, ETIMEOUT)


def test_a_rank_that_leaves_between_calls(pkg, lib):
    status, digest, done, _ = loopback(pkg, lib, [8] * 4, calls=6, wait_us=50000, faults=[(LEAVE, 2, 4, -1)])
    assert status[2] == OK and done[2] == 3               # left cleanly after three calls
    for r in (0, 1, 3):
        assert status[r] == ETIMEOUT and done[r] == 3     # call 4 never completes, nobody hangs
    rows = np.array([8] * 4, np.int32)
    for r in range(4):                                    # what was completed is correct
        assert digest[r] == lib.iris_b200_ring_loopback_digest(4, rows.ctypes.data, 96, 3, r)


def test_argument_checks(lib):
    rows = np.array([4, 0], np.int32)
    out = np.zeros(2, np.int32)
    dig = np.zeros(2, np.uint64)
    assert lib.iris_b200_ring_loopback(2, rows.ctypes.data, 8, 1, 0, None, 0, out.ctypes.data, dig.ctypes.data,
                                       out.ctypes.data) == 1
    assert lib.iris_b200_ring_loopback(0, rows.ctypes.data, 8, 1, 0, None, 0, out.ctypes.data, dig.ctypes.data,
                                       out.ctypes.data) == 1
