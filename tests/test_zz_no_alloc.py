"""The allocation-free attention entry point against the ordinary one.

Collected last on purpose: a failure here must not hide the other tests from
a run that stops at the first failure. Runs alone in a fresh process as well
as after the rest of the suite (it initialises the device itself)."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu

D = 128


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    lib = ge.load_package().load()
    lib.init()
    yield lib
    lib.check()


def test_no_alloc_split_k_matches_plain_attention_twice_in_a_row(lib):
    """Callers that may not touch the allocator (real-time threads, hosts with
    a fully committed memory budget) get the same numbers as everyone else:
    two back-to-back calls on different inputs, sharing the built-in scratch,
    each compared with iris_dev_attention on the same inputs."""
    H, sq, sk = 6, 700, 1500
    dout_a = lib.alloc(sq * H * D * 2)
    dout_b = lib.alloc(sq * H * D * 2)
    results = []
    for call, nsplit in enumerate((3, 5)):
        q, k, v = (ol.to_bf16(ol.randn(90 + 3 * call + i, n, H * D)) for i, n in enumerate((sq, sk, sk)))
        dq, dk, dv = lib.to_device(q), lib.to_device(k), lib.to_device(v)
        lib.iris_dev_attention(dout_a, H * D, dq, dk, dv, H * D, sq, sk, H, H, D, 1.0 / np.sqrt(D), 0, None)
        rc = lib.iris_b200_attention_noalloc(dout_b, H * D, dq, dk, dv, H * D, sq, sk, H, 1.0 / np.sqrt(D), nsplit)
        assert rc == 0, rc
        want = ol.from_bf16(lib.to_host(dout_a, (sq, H * D), np.uint16))
        got = ol.from_bf16(lib.to_host(dout_b, (sq, H * D), np.uint16))
        lib.check()
        for p in (dq, dk, dv):
            lib.iris_dev_free(p)
        mx, cs = ol.compare_heads(got, want, H)
        assert np.isfinite(got).all()
        # same tolerance as the parity gate of the other attention tests
        assert mx.max() <= 2e-2 and cs.min() >= 0.9999, (call, mx, cs)
        # and both against the CPU oracle, so that the two entry points cannot agree on a wrong answer
        truth = ol.dev_attention(ol.from_bf16(q), ol.from_bf16(k), ol.from_bf16(v), H)
        for res in (got, want):
            mx, cs = ol.compare_heads(res, truth, H)
            assert mx.max() <= 2e-2 and cs.min() >= 0.9999, (call, mx, cs)
        results.append(got)
    assert not np.array_equal(results[0], results[1])
    lib.iris_dev_free(dout_a)
    lib.iris_dev_free(dout_b)


def test_no_alloc_rejects_what_does_not_fit(lib):
    limit = lib.iris_b200_attention_noalloc_max_elems()
    assert limit == 4 << 20
    rows = limit // (32 * D) + 1                  # one row too many for 32 heads
    rc = lib.iris_b200_attention_noalloc(256, 32 * D, 256, 256, 256, 32 * D, rows, 128, 32, 0.1, 2)
    assert rc == 1                                # IRIS_B200_EINVAL, nothing launched
    lib.iris_b200_clear_error()
    assert lib.iris_b200_attention_noalloc(256, 2 * D, 256, 256, 256, 2 * D, 10, 128, 2, 0.1, 0) == 1
    lib.iris_b200_clear_error()
    # row strides shorter than a row of heads: the output would run past its buffer, the inputs overlap
    assert lib.iris_b200_attention_noalloc(256, 2 * D - 8, 256, 256, 256, 2 * D, 10, 128, 2, 0.1, 2) == 1
    lib.iris_b200_clear_error()
    assert lib.iris_b200_attention_noalloc(256, 2 * D, 256, 256, 256, 2 * D - 8, 10, 128, 2, 0.1, 2) == 1
    lib.iris_b200_clear_error()
