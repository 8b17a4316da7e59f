"""zn_accumulate_bias_noalloc against zn_accumulate_bias.

The no-allocation entry point serves programs that cannot let this library call cudaMalloc (their own pool
owns the device memory, or they cannot take the stall an allocation causes).  It must give what the regular
entry point gives.  The file name sorts last on purpose: if it fails, a run that stops at the first failure
has already run every other test.  It works on its own in a fresh process as well as after the other tests:
the fixed scratch block it uses needs no preparation and keeps no state that matters between calls.
"""
import numpy as np
import pytest

import zigneuron_b200 as zn

pytestmark = pytest.mark.gpu


def test_noalloc_bias_accumulation_matches_regular_entry_point():
    be = zn.Backend(0, zn.Precision.FP32_SIMT)
    rng = np.random.default_rng(21)
    # two calls in a row; the second is smaller, so stale partial sums of the first stay in the shared block
    for rows, cols in [(4097, 513), (300, 70)]:
        g = rng.standard_normal((rows, cols)).astype(np.float32)
        gb0 = rng.standard_normal(cols).astype(np.float32)
        dg = be.tensor(g)
        want_t, got_t = be.tensor(gb0), be.tensor(gb0)
        be.accumulateBias(want_t, dg)              # existing entry point (context scratch, may allocate)
        be.accumulateBiasNoAlloc(got_t, dg)        # new entry point (fixed block, allocates nothing)
        be.endCommandBatch()
        want, got = want_t.numpy(), got_t.numpy()
        # same kernels, same split of the rows: the tolerance of the other bias tests (1e-5 of the term size) holds with room
        assert np.max(np.abs(got - want)) <= 1e-5 * max(1.0, np.sqrt(rows)) * np.max(np.abs(g)), (rows, cols)
        assert np.array_equal(got, want), (rows, cols)
        for t in (dg, want_t, got_t):
            t.free()
    be.deinit()


def test_noalloc_follows_the_exact_mode_of_the_context():
    """On a FP32_EXACT context the regular entry point adds each column's rows in ascending order (the reference's
    cpuAccumulateBias); the no-allocation entry point must do the same, bit for bit, on two calls in a row."""
    be = zn.Backend(0, zn.Precision.FP32_EXACT)
    rng = np.random.default_rng(22)
    for rows, cols in [(1500, 257), (65, 1030)]:
        g = rng.standard_normal((rows, cols)).astype(np.float32)
        gb0 = rng.standard_normal(cols).astype(np.float32)
        dg = be.tensor(g)
        want_t, got_t = be.tensor(gb0), be.tensor(gb0)
        be.accumulateBias(want_t, dg)
        be.accumulateBiasNoAlloc(got_t, dg)
        be.endCommandBatch()
        want, got = want_t.numpy(), got_t.numpy()
        seq = gb0.copy()
        for r in range(rows):                       # the reference's order: gb[c] += g[r][c], r ascending
            seq += g[r]
        assert np.array_equal(want, seq), (rows, cols)
        assert np.array_equal(got, want), (rows, cols)
        for t in (dg, want_t, got_t):
            t.free()
    be.deinit()


def test_noalloc_rejects_what_does_not_fit_and_host_pointers():
    be = zn.Backend(0)
    cols = 1_100_000                                # one row: 1 split x 1.1e6 columns > 1,048,576 floats of scratch
    g, gb = be.tensor(cols), be.tensor(cols)
    with pytest.raises(zn.ZnError) as ei:
        be.accumulateBiasNoAlloc(gb, g)
    assert ei.value.status == 1 and "fixed block" in str(ei.value)
    with pytest.raises(zn.ZnError):                 # host memory would need a staging allocation
        be.accumulateBiasNoAlloc(np.zeros(4, np.float32), np.zeros(8, np.float32))
    g.free()
    gb.free()
    be.deinit()
