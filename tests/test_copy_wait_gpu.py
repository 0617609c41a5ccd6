"""Failure detection of the input copies.  A world waits a bounded number of polls
for its TMA bulk copies; when the wait runs out it reports through bit 30 of its
``overflow`` word, writes no result, and the context stays usable.  The failure is
injected from the host (imn_set_copy_wait_limit): no copy is issued while the barrier
still expects bytes, so the wait runs out with nothing in flight.  No GPU fault, trap
or hang is involved."""

import copy

import numpy as np
import pytest

from instantmimic_b200 import _lib, mjw_model, synthetic
from instantmimic_b200 import mjw_step_optimized as runtime

from helpers import run_oracle

pytestmark = pytest.mark.gpu

COPY_TIMEOUT = 1 << 30


def _solve(md, dd, scratch):
    import torch

    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)
    torch.cuda.synchronize()
    return mjw_model.to_host(dd)


@pytest.mark.parametrize("name,withhold", [("humanoid", 1), ("snu", 1), ("snu", 2)])
def test_copy_wait_runs_out_and_the_next_solve_is_clean(oracle, cuda_device, name, withhold):
    m, d, _ = synthetic.make_workload(name, 48, seed=5, rowless_fraction=0.1)
    md, dd = mjw_model.to_device(m, cuda_device), mjw_model.to_device(copy.deepcopy(d), cuda_device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, cuda_device)
    lib = _lib.lib()
    dd.qacc.fill_(123.0)
    try:
        assert lib.imn_set_copy_wait_limit(16, withhold) == 0
        got = _solve(md, dd, scratch)
    finally:
        assert lib.imn_set_copy_wait_limit(1 << 22, 0) == 0
    # withhold bit 0: the initial load of every world; bit 1: the row tiles, which only
    # worlds with rows fetch
    hit = np.ones(d.nworld, bool) if withhold == 1 else d.nefc > 0
    assert ((got.overflow & COPY_TIMEOUT) != 0).tolist() == hit.tolist()
    assert (got.qacc[hit] == 123.0).all()  # no result was written for the lost worlds
    # same buffers, default limit: the solve is the oracle's again
    dd.overflow.zero_()
    got = _solve(md, dd, scratch)
    want, _, _ = run_oracle(oracle, m, d)
    np.testing.assert_array_equal(got.overflow, want.overflow)
    np.testing.assert_array_equal(got.solver_niter, want.solver_niter)
    np.testing.assert_array_equal(got.qacc.view(np.uint32), want.qacc.view(np.uint32))
