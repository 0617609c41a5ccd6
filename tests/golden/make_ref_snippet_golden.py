"""Writes ref_snippets.npz:  python tests/golden/make_ref_snippet_golden.py [out.npz]   (needs a GPU)

Golden input / output vectors of the REFERENCE'S OWN CUDA text for the sparse-pattern
Hessian factor and the tree L'DL of M, run on a B200.  oracle/ref_snippets.py asks the
reference's generators for that text, wraps it and compiles it with nvcc (defaults, i.e.
fused multiply-add contraction on, as Warp compiles it) into
oracle/_ref/libref_snippets.so; this script drives that library on seeded inputs and
stores what went in and what came out:

  tree       x = M^-1 y                                  (tree_ldl.py:194-383)
  init       packed H | N | 1/D, search, sums            (sparse_hessian.py:571-637)
  update     flipped rows -> packed H, search, sums      (:483-527, factor levels :410-452)
  resident   solve with the factor kept in U             (:528-547)
  nonfused   factor of the dense H, then a solve-only call (:651-676)

for the models of oracle/ref_snippets.case_models.  The file is committed; the tests
replay it on the CPU oracle and on the CUDA kernels bit for bit, with no reference tree
and no _ref library present.
"""

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from instantmimic_b200 import synthetic  # noqa: E402
from oracle import ref_snippets  # noqa: E402

W = 6
QUADRATIC = 1


def inputs(name: str, case: dict, groups):
    """Seeded inputs of one case: a solver batch of the model with a plausible active set,
    a flip of a few rows, fresh gradients."""
    rng = np.random.default_rng(100 + case["index"])
    if name == "limbs64":
        m, d, Mdense = synthetic.make_sweep_point(64, 32, W, seed=3, couple=False)
    else:
        m, d, Mdense = synthetic.make_workload(name.split("_")[0], W, seed=3)
    if name.endswith("_pairs"):
        d.efc.J[:] = ref_snippets.rows_for_groups(m, groups, W, d.njmax, rng)
    nv, R, P = m.nv, d.njmax, m.nv_pad
    nefc = np.minimum(d.nefc, R).astype(np.int32)
    live = np.arange(R)[None, :] < nefc[:, None]
    state = np.where(live & (rng.random((W, R)) < 0.6), QUADRATIC, 0).astype(np.int32)
    ids = np.zeros((W, R), np.int32)
    count = np.zeros(W, np.int32)
    uni = np.zeros((W, nv + 1), np.int32)
    state2 = state.copy()
    for w in range(W):
        rows = np.flatnonzero(live[w])
        k = min(len(rows), int(rng.integers(0, 5)))  # world 0.. some with no flip at all
        flip = np.sort(rng.choice(rows, size=k, replace=False)) if k else np.zeros(0, np.int64)
        state2[w, flip] = np.where(state[w, flip] == QUADRATIC, 0, QUADRATIC)
        ids[w, :k], count[w] = flip, k
        dofs = np.flatnonzero((d.efc.J[w, flip] != 0).any(axis=0)) if k else np.zeros(0, np.int64)
        uni[w, : len(dofs)], uni[w, nv] = dofs, len(dofs)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)  # noqa: E731
    H = Mdense.astype(np.float64).copy() if Mdense is not None else None
    dense = np.zeros((W, P, P), np.float32)
    Jq = d.efc.J.astype(np.float64) * (state == QUADRATIC)[..., None]
    full = np.einsum("wra,wr,wrb->wab", Jq, d.efc.D.astype(np.float64), d.efc.J.astype(np.float64))
    dense[:, :nv, :nv] = (H + full).astype(np.float32)
    return m, {
        "J": f32(d.efc.J), "D": f32(d.efc.D), "state": state, "state2": state2, "nefc": nefc, "M": f32(d.M),
        "ids": ids, "count": count, "uni": uni, "H": dense,
        "grad": f32(np.pad(rng.normal(size=(3, W, nv)), ((0, 0), (0, 0), (0, P - nv)))),
        "y": f32(rng.normal(size=(W, nv))),
    }


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE / "ref_snippets.npz"
    lib = C.CDLL(str(ref_snippets.LIB))
    dev = torch.device("cuda:0")
    out = {}
    groups_of = {name: groups for name, _, groups in ref_snippets.case_models()}
    for case in ref_snippets.manifest():
        name, c, nv, P = case["name"], case["index"], case["nv"], case["nv_pad"]
        m, x = inputs(name, case, groups_of[name])
        R = x["J"].shape[1]
        t = {k: torch.from_numpy(v).to(dev) for k, v in x.items()}
        ptr = lambda a: C.c_void_p(a.data_ptr())  # noqa: E731
        z = lambda *s: torch.zeros(*s, device=dev)  # noqa: E731
        done = torch.zeros(W, dtype=torch.uint8, device=dev)
        for k, v in x.items():
            out[f"{name}/in/{k}"] = v

        def keep(tag, U, search, sd, dec):
            torch.cuda.synchronize()
            out[f"{name}/{tag}/U"] = U.cpu().numpy().copy()
            out[f"{name}/{tag}/search"] = search.cpu().numpy().copy()
            out[f"{name}/{tag}/search_dot"] = sd.cpu().numpy().copy()
            out[f"{name}/{tag}/decrement"] = dec.cpu().numpy().copy()

        # tree L'DL
        xs = z(W, nv)
        assert lib.ref_tree_ldl(c, ptr(t["M"]), case["nM"], ptr(t["y"]), ptr(xs), W, None) == 0
        torch.cuda.synchronize()
        out[f"{name}/tree/x"] = xs.cpu().numpy().copy()
        # fused: initial assembly, then an update with flipped rows, then a resident solve
        U, search, sd, dec = z(W, P, P), z(W, nv), z(W), z(W)
        assert lib.ref_sparse_init(c, ptr(done), ptr(t["nefc"]), ptr(t["J"]), R, ptr(t["D"]), ptr(t["state"]),
                                   ptr(t["M"]), case["nM"], ptr(t["grad"][0]), P, ptr(U), ptr(search), ptr(sd),
                                   ptr(dec), W, None) == 0
        keep("init", U, search, sd, dec)
        assert lib.ref_sparse_fused(c, ptr(t["J"]), R, ptr(t["D"]), ptr(t["state2"]), ptr(t["ids"]), ptr(t["count"]),
                                    ptr(t["uni"]), ptr(t["grad"][1]), P, ptr(U), ptr(search), ptr(sd), ptr(dec), 0, W,
                                    None) == 0
        keep("update", U, search, sd, dec)
        U.copy_(torch.from_numpy(out[f"{name}/init/U"]))
        assert lib.ref_sparse_fused(c, ptr(t["J"]), R, ptr(t["D"]), ptr(t["state"]), ptr(t["ids"]), ptr(t["count"]),
                                    ptr(t["uni"]), ptr(t["grad"][2]), P, ptr(U), ptr(search), ptr(sd), ptr(dec), 1, W,
                                    None) == 0
        keep("resident", U, search, sd, dec)
        # non-fused: factor the dense H, then a solve-only call with another gradient
        U, search, sd, dec = z(W, P, P), z(W, nv), z(W), z(W)
        changed = torch.ones(W, dtype=torch.int32, device=dev)
        assert lib.ref_sparse_nonfused(c, ptr(done), ptr(t["grad"][0]), P, ptr(t["H"]), ptr(changed), ptr(changed),
                                       ptr(U), ptr(search), ptr(sd), ptr(dec), 0, 0, W, None) == 0
        keep("nonfused_factor", U, search, sd, dec)
        changed.zero_()
        assert lib.ref_sparse_nonfused(c, ptr(done), ptr(t["grad"][1]), P, ptr(t["H"]), ptr(changed), ptr(changed),
                                       ptr(U), ptr(search), ptr(sd), ptr(dec), 1, 0, W, None) == 0
        keep("nonfused_solve", U, search, sd, dec)
    out["names"] = np.asarray([c["name"] for c in ref_snippets.manifest()])
    np.savez_compressed(out_path, **out)
    print(len(out), "arrays,", out_path.stat().st_size, "bytes ->", out_path)


if __name__ == "__main__":
    main()
