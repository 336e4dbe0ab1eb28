"""Attention over key runs (the launch a ring call makes), the key split into
several parts, and the failure paths of the bounded waits, on one GPU.

The failure tests make a wait run out from the host: an arrival word that
nobody advances, an arrival ticket that nobody took. Nothing faults or hangs:
the launch returns at the wait limit (set to a few milliseconds here), the
status word reports IRIS_B200_ETIMEOUT and the next call is correct again."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu

D = 128
MAX_ABS, MIN_COS = 2e-2, 0.9999
ETIMEOUT, ECHECK = 3, 9


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.iris_b200_set_wait_limit_us(0)
    lib.check()


def key_runs(runs):
    import __graft_entry__ as ge
    KeyRun = ge.load_package().binding.KeyRun
    arr = (KeyRun * len(runs))()
    for i, (view, row0, rows, arrive) in enumerate(runs):
        arr[i].view, arr[i].row0, arr[i].rows, arr[i].arrive = view, row0, rows, arrive
    return arr


class Problem:
    """Queries, and keys scattered as runs over two buffers with different
    row strides: view 0 is a fused [rows, 3 H D] activation (K and V are
    column slices), view 1 a slot pool [rows, 2 H D] (K | V)."""

    def __init__(self, lib, H, sq, run_rows, seed, views=None, gaps=(5, 11)):
        self.lib, self.H, self.sq = lib, H, sq
        hd = H * D
        self.q = ol.to_bf16(ol.randn(seed, sq, hd))
        views = views or [i % 2 for i in range(len(run_rows))]
        sizes = [0, 0]
        self.runs = []
        for n, vw in zip(run_rows, views):
            sizes[vw] += gaps[vw]                       # rows between runs that belong to nobody
            self.runs.append([vw, sizes[vw], n, -1])
            sizes[vw] += n
        self.bufs = [ol.to_bf16(ol.randn(seed + 1, max(sizes[0], 1), 3 * hd)),
                     ol.to_bf16(ol.randn(seed + 2, max(sizes[1], 1), 2 * hd))]
        ks, vs = [], []
        for vw, r0, n, _ in self.runs:
            b = self.bufs[vw]
            ks.append(b[r0:r0 + n, hd:2 * hd] if vw == 0 else b[r0:r0 + n, :hd])
            vs.append(b[r0:r0 + n, 2 * hd:] if vw == 0 else b[r0:r0 + n, hd:])
        self.k, self.v = np.concatenate(ks), np.concatenate(vs)
        self.dq = lib.to_device(self.q)
        self.dbuf = [lib.to_device(b) for b in self.bufs]
        self.dout = lib.to_device(np.full((sq, hd), 0x7FC0, np.uint16))      # NaN canaries

    def want(self):
        return ol.dev_attention(ol.from_bf16(self.q), ol.from_bf16(self.k), ol.from_bf16(self.v), self.H)

    def launch(self, nparts=0, words=None, value=0):
        hd = self.H * D
        b0, b1 = self.dbuf
        runs = key_runs(self.runs)
        return self.lib.iris_b200_attention_runs(
            self.dout, hd, self.dq, hd, self.sq, self.H, 1.0 / np.sqrt(D),
            b0 + hd * 2, b0 + 2 * hd * 2, 3 * hd, b1, b1 + hd * 2, 2 * hd,
            runs, len(self.runs), words, value, nparts)

    def result(self):
        return ol.from_bf16(self.lib.to_host(self.dout, (self.sq, self.H * D), np.uint16))

    def free(self):
        for p in [self.dq, self.dout] + self.dbuf:
            self.lib.iris_dev_free(p)


def check(got, want, H):
    assert np.isfinite(got).all()
    mx, cs = ol.compare_heads(got, want, H)
    assert mx.max() <= MAX_ABS and cs.min() >= MIN_COS, (mx, cs)


@pytest.mark.parametrize("nparts", [0, 1, 2, 3, 5, 8])
def test_runs_over_two_buffers_equal_one_sequence(lib, nparts):
    """Runs of ragged lengths (partial last tiles in the middle of the key
    sequence), alternating between the two views, cut into 1..8 parts."""
    pr = Problem(lib, 3, 300, [130, 257, 64, 1, 511, 128, 300, 77], seed=100)
    try:
        assert pr.launch(nparts) == 0
        got = pr.result()
        lib.check()
        check(got, pr.want(), 3)
    finally:
        pr.free()


def test_many_query_blocks_and_parts_share_the_work_list(lib):
    """More work items than SMs (dynamic work list over several rounds) with
    a forced four-way key split and a last query block of a single tile."""
    H, sq = 4, 256 * 9 + 70
    pr = Problem(lib, H, sq, [512, 640, 384, 512], seed=110, views=[0, 1, 1, 1])
    try:
        for nparts in (4, 2):
            assert pr.launch(nparts) == 0
            got = pr.result()
            lib.check()
            check(got, pr.want(), H)
    finally:
        pr.free()


def test_runs_wait_for_their_arrival_words(lib):
    """Words already at (or beyond) the call's value let the launch through,
    whatever garbage other words hold; the comparison is wrap-around safe."""
    pr = Problem(lib, 2, 200, [256, 200, 300], seed=120, views=[0, 1, 1])
    pr.runs[1][3], pr.runs[2][3] = 3, 7
    words = np.zeros(32, np.uint32)
    words[3], words[7] = 0xFFFFFFF0, 0x00000002            # value 0xFFFFFFF0: 3 equal, 7 ahead after the wrap
    dwords = lib.to_device(words)
    try:
        assert pr.launch(2, dwords, 0xFFFFFFF0) == 0
        got = pr.result()
        lib.check()
        check(got, pr.want(), 2)
    finally:
        lib.iris_dev_free(dwords)
        pr.free()


def test_arrival_that_never_comes_times_out_and_the_next_call_is_fine(lib):
    pr = Problem(lib, 2, 300, [256, 256], seed=130, views=[0, 1])
    pr.runs[1][3] = 5
    dwords = lib.to_device(np.zeros(32, np.uint32))        # word 5 stays at 0, the call wants 9
    try:
        lib.iris_b200_set_wait_limit_us(5000)
        assert pr.launch(0, dwords, 9) == 0                # the launch itself is accepted
        assert lib.iris_b200_check_device_status() == ETIMEOUT
        lib.iris_b200_clear_error()
        lib.iris_b200_set_wait_limit_us(0)
        # the same problem with the word in place, then an unrelated plain call
        lib.iris_dev_upload(dwords, np.full(32, 9, np.uint32).ctypes.data, 128)
        assert pr.launch(0, dwords, 9) == 0
        got = pr.result()
        lib.check()
        check(got, pr.want(), 2)
    finally:
        lib.iris_b200_set_wait_limit_us(0)
        lib.iris_dev_free(dwords)
        pr.free()


def test_stale_split_ticket_times_out_and_the_scratch_recovers(lib):
    """Host-side fault injection: a ticket nobody took makes the parts of one
    query block wait for a partial that never comes."""
    pr = Problem(lib, 2, 256, [384, 384], seed=140, views=[0, 0], gaps=(0, 0))
    try:
        assert pr.launch(2) == 0
        lib.check()
        want = pr.want()
        check(pr.result(), want, 2)
        lib.iris_b200_set_wait_limit_us(5000)
        assert lib.iris_b200_inject_fault(1) == 0
        assert pr.launch(2) == 0
        # the self-checking build (-DIRIS_B200_CHECK) sees the impossible ticket first
        assert lib.iris_b200_check_device_status() in (ETIMEOUT, ECHECK)
        lib.iris_b200_clear_error()
        lib.iris_b200_set_wait_limit_us(0)
        for nparts in (2, 3, 0):                           # tickets and work-list counters are clean again
            lib.iris_dev_upload(pr.dout, np.full((256, 2 * D), 0x7FC0, np.uint16).ctypes.data, 256 * 2 * D * 2)
            assert pr.launch(nparts) == 0
            got = pr.result()
            lib.check()
            check(got, want, 2)
    finally:
        lib.iris_b200_set_wait_limit_us(0)
        pr.free()


def test_run_argument_checks(lib):
    pr = Problem(lib, 2, 64, [128], seed=150, views=[0])
    try:
        hd = 2 * D
        runs = key_runs([(2, 0, 128, -1)])                                   # no such view
        assert lib.iris_b200_attention_runs(pr.dout, hd, pr.dq, hd, 64, 2, 0.1, pr.dbuf[0], pr.dbuf[0], 3 * hd,
                                            None, None, 0, runs, 1, None, 0, 0) == 1
        lib.iris_b200_clear_error()
        runs = key_runs([(0, 0, 128, 4)])                                    # guarded run without words
        assert lib.iris_b200_attention_runs(pr.dout, hd, pr.dq, hd, 64, 2, 0.1, pr.dbuf[0], pr.dbuf[0], 3 * hd,
                                            None, None, 0, runs, 1, None, 0, 0) == 1
        lib.iris_b200_clear_error()
        runs = key_runs([(0, 0, 128, -1)])                                   # output stride shorter than a row
        assert lib.iris_b200_attention_runs(pr.dout, hd - 8, pr.dq, hd, 64, 2, 0.1, pr.dbuf[0], pr.dbuf[0], 3 * hd,
                                            None, None, 0, runs, 1, None, 0, 0) == 1
        lib.iris_b200_clear_error()
        assert lib.iris_b200_inject_fault(99) == 1
    finally:
        pr.free()
