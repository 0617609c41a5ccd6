"""Shared helpers of the parity tests."""

from __future__ import annotations

import copy
from types import SimpleNamespace

import numpy as np

from instantmimic_b200 import mjw_model


def host_ctx(m, d, matrices=True):
    W, nv, R, P = d.nworld, m.nv, d.njmax, m.nv_pad
    f = lambda *s: np.zeros(s, np.float32)  # noqa: E731
    i = lambda *s: np.zeros(s, np.int32)  # noqa: E731
    return SimpleNamespace(
        Jaref=f(W, R), jv=f(W, R), search=f(W, nv), mv=f(W, nv), grad=f(W, P),
        h=f(W, P, P) if matrices else None, hfactor=f(W, P, P) if matrices else None,
        search_dot=f(W), grad_dot=f(W), grad_scale=f(W), newton_decrement=f(W),
        improvement=f(W), alpha=f(W),
        done=np.zeros(W, np.uint8), search_unchanged=np.zeros(W, np.uint8),
        ls_exhausted=np.zeros(W, np.uint8),
        quad_changed_ids=i(W, R), quad_changed_count=i(W), state_changed_count=i(W),
        newton_dof_union=i(W, nv + 1), stats=i(W, 4),
    )


def run_oracle(oracle, m, d, matrices=True, threads=0):
    """Solve a copy of host data with the oracle; returns (data, ctx, nsolving)."""
    d2 = copy.deepcopy(d)
    ctx = host_ctx(m, d2, matrices)
    nsolving = np.zeros(1, np.int32)
    oracle.solve(m, d2, ctx, nsolving, threads=threads)
    return d2, ctx, nsolving


def run_cuda(m, d, device, matrices=True, use_optimized_kernel=True, ordered=True):
    """Solve a copy of host data on the GPU through solve_with_scratch; results on host.
    ``ordered=False`` withholds the context's world-order scratch, so worlds are handed
    to the GPU in index order instead of by descending row count."""
    import torch

    from instantmimic_b200 import mjw_step_optimized as runtime

    md = mjw_model.to_device(m, device)
    dd = mjw_model.to_device(copy.deepcopy(d), device)
    scratch = runtime.make_optimized_fwd_position_scratch(md, dd, device, with_matrices=matrices, with_stats=matrices)
    if not ordered and scratch.solver_context is not None:
        scratch.solver_context.world_order = None
    runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=use_optimized_kernel)
    torch.cuda.synchronize()
    ctx = scratch.solver_context
    hctx = SimpleNamespace(
        **{k: (v.cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in vars(ctx).items()}
    ) if ctx is not None else None
    nsolving = scratch.solver_nsolving.cpu().numpy() if scratch.solver_nsolving is not None else None
    return mjw_model.to_host(dd), hctx, nsolving, (md, dd, scratch)


def scaled_err(a, b):
    """The reference's parity norm (tests/test_mjw_newton_fusion.py:217-226)."""
    a = a.astype(np.float64).reshape(a.shape[0], -1)
    b = b.astype(np.float64).reshape(b.shape[0], -1)
    return float(np.max(np.linalg.norm(a - b, axis=1) / np.maximum(1.0, np.linalg.norm(b, axis=1))))


def reference_f64(m, d, Mdense, iters=200):
    """Independent float64 primal Newton solver with exact line search by
    bisection on the derivative; returns qacc (W, nv).  Written without looking at
    operation order: it only shares the problem statement with the oracle."""
    W, nv = d.nworld, m.nv
    out = np.zeros((W, nv))
    for w in range(W):
        n = min(int(d.nefc[w]), d.njmax)
        ne, nf = int(d.ne[w]), int(d.nf[w])
        M = Mdense[w].astype(np.float64)
        qs = d.qfrc_smooth[w].astype(np.float64)
        if n == 0:
            out[w] = d.qacc_smooth[w]
            continue
        J = d.efc.J[w, :n].astype(np.float64)
        D = d.efc.D[w, :n].astype(np.float64)
        aref = d.efc.aref[w, :n].astype(np.float64)
        fl = d.efc.frictionloss[w, :n].astype(np.float64)
        kind = np.full(n, 2)
        kind[:ne] = 0
        kind[ne:ne + nf] = 1

        def rows(x):
            """force, active-quadratic mask, cost"""
            f = np.zeros(n); q = np.zeros(n, bool); c = np.zeros(n)
            for r in range(n):
                if kind[r] == 0:
                    f[r], q[r], c[r] = -D[r] * x[r], True, 0.5 * D[r] * x[r] ** 2
                elif kind[r] == 1:
                    rf = fl[r] / D[r]
                    if x[r] <= -rf:
                        f[r], c[r] = fl[r], fl[r] * (-0.5 * rf - x[r])
                    elif x[r] >= rf:
                        f[r], c[r] = -fl[r], fl[r] * (-0.5 * rf + x[r])
                    else:
                        f[r], q[r], c[r] = -D[r] * x[r], True, 0.5 * D[r] * x[r] ** 2
                elif x[r] < 0:
                    f[r], q[r], c[r] = -D[r] * x[r], True, 0.5 * D[r] * x[r] ** 2
            return f, q, c

        qa = d.qacc_smooth[w].astype(np.float64).copy()
        a0 = np.linalg.solve(M, qs)

        def cost(q):
            x = J @ q - aref
            _, _, c = rows(x)
            dq = q - a0
            return 0.5 * dq @ M @ dq + c.sum()

        for _ in range(iters):
            x = J @ qa - aref
            f, q, _ = rows(x)
            g = M @ qa - qs - J.T @ f
            if np.linalg.norm(g) < 1e-11 * max(1.0, np.linalg.norm(qs)):
                break
            H = M + (J[q].T * D[q]) @ J[q]
            s = -np.linalg.solve(H, g)
            # exact line search: derivative is monotone in alpha
            def dphi(al):
                xx = J @ (qa + al * s) - aref
                ff, _, _ = rows(xx)
                return s @ (M @ (qa + al * s) - qs - J.T @ ff)
            lo, hi = 0.0, 1.0
            while dphi(hi) < 0 and hi < 1e6:
                hi *= 2
            for _ in range(200):
                mid = 0.5 * (lo + hi)
                if dphi(mid) < 0:
                    lo = mid
                else:
                    hi = mid
            qa = qa + 0.5 * (lo + hi) * s
        out[w] = qa
    return out
