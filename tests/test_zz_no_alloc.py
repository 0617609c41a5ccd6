"""The allocation-free factor + solve entry point.

``imn_blocked_dense_factor_solve_static`` serves callers that cannot hand the
library a factor workspace because they are not allowed to allocate device memory
at the call site (a step under CUDA-graph capture, a process whose device memory
is owned by another framework's pool, a host that forbids cudaMalloc after
start-up).  Its workspace is a fixed array inside the library.  The test calls it
through the C ABI twice in a row and requires the same bits as the ordinary entry
point with a caller-owned workspace; the second call also runs on a different
batch so that a stale factor left in the shared array would show.

The file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""

import ctypes as C

import numpy as np
import pytest

from instantmimic_b200 import abi, synthetic
from instantmimic_b200.mjw_kernels import indexed_factor
from instantmimic_b200.mjw_model import make_data, put_model, to_device

pytestmark = pytest.mark.gpu


def _case(nv, worlds, rhs, seed):
    parent, body = synthetic.limb_tree(nv)
    m = put_model(parent, body_of_dof=body)
    rng = np.random.default_rng(seed)
    Mv, _ = synthetic.random_mass_matrices(m, worlds, rng)
    y = rng.normal(size=(worlds, nv, rhs)).astype(np.float32)
    return m, Mv, y


def test_static_workspace_entry_matches_caller_workspace_entry_twice(cuda_device):
    import torch

    from instantmimic_b200 import _lib

    lib = _lib.lib()
    stream = _lib.current_stream_handle()
    nv, worlds, rhs = 35, 40, 2
    m, _, _ = _case(nv, worlds, rhs, 0)
    md = to_device(m, cuda_device)
    dd = to_device(make_data(m, worlds, 4), cuda_device)
    scratch = indexed_factor.create_blocked_dense_factor_solve_scratch(md, dd, cuda_device)
    plan = scratch.struct
    active = torch.ones(worlds, dtype=torch.int32, device=cuda_device)
    active[5] = 0
    for seed in (11, 12):  # two calls in a row, different matrices
        _, Mv, y = _case(nv, worlds, rhs, seed)
        Mt = torch.from_numpy(Mv).to(cuda_device)
        yt = torch.from_numpy(y).to(cuda_device)
        want = torch.full_like(yt, -3.0)
        got = torch.full_like(yt, -3.0)
        U = torch.zeros((worlds, scratch.pad, scratch.pad), dtype=torch.float32, device=cuda_device)
        rc = lib.imn_blocked_dense_factor_solve(
            C.byref(plan), Mt.data_ptr(), Mt.stride(0), yt.data_ptr(), U.data_ptr(), want.data_ptr(),
            active.data_ptr(), worlds, rhs, 0, stream)
        assert rc == 0, lib.imn_last_error()
        rc = lib.imn_blocked_dense_factor_solve_static(
            C.byref(plan), Mt.data_ptr(), Mt.stride(0), yt.data_ptr(), got.data_ptr(), active.data_ptr(),
            worlds, rhs, stream)
        assert rc == 0, lib.imn_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        np.testing.assert_array_equal(got.cpu().numpy(), want.cpu().numpy())
        np.testing.assert_array_equal(got[5].cpu().numpy(), -3.0)  # inactive world untouched


def test_static_workspace_entry_rejects_sizes_beyond_its_array(cuda_device):
    from instantmimic_b200 import _lib

    lib = _lib.lib()
    plan = abi.ImnBlockedPlan()
    plan.nv, plan.pad, plan.nM = 70, 80, 10
    too_many = 8 * 1024 * 1024 // (80 * 80) + 1
    rc = lib.imn_blocked_dense_factor_solve_static(C.byref(plan), None, 0, None, None, None, too_many, 1, None)
    assert rc == abi.IMN_ERR_LIMIT
    assert b"exceed" in lib.imn_last_error()
