"""The CPU baseline of the benchmark is the reference's own vectorized engine (oracle/_ref/libdaphne_ref_engine.so).
Its results must be those of the reference's kernels called one after the other: the engine only partitions rows."""
import numpy as np
import pytest

from oracle import cpu_pipelines, refengine, refkernels

pytestmark = pytest.mark.skipif(not (refengine.available() and refkernels.available()),
                                reason="the reference-built engine / kernels are not present")


@pytest.mark.parametrize("rows,threads", [(1234, 3), (50000, 8), (7, 4)])
def test_engine_equals_the_kernel_sequence(rows, threads):
    x = 5.0 + 2.0 * np.random.default_rng(rows).standard_normal((rows, 32))
    mu, sd, r, s, m, idx = cpu_pipelines.standardise_aggregate(x, threads=1, k=refkernels)
    for vectorized in (True, False):
        e_mu, e_sd, e_r, e_s, e_m, e_idx, ms = refengine.standardise_aggregate(x, threads, vectorized)
        assert np.array_equal(e_mu, mu) and np.array_equal(e_sd, sd)
        assert np.array_equal(e_r, r) and np.array_equal(e_m, m) and np.array_equal(e_idx, idx)
        assert abs(e_s - s) <= 1e-12 * abs(s)  # the ADD combine of the task partials regroups the sum
        assert ms[3] > 0.0
