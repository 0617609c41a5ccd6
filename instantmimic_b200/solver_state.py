"""Solver-state files: everything one ``solve_with_scratch`` call reads and writes, as
one ``.npz``.

Purpose.  The Newton solve sits in the middle of a physics step whose other stages
(kinematics, constraint rows, M) come from mujoco-warp.  A state file freezes the
solver-facing arrays of ``Model`` and ``Data`` at the call
(src/instantmimic/utils/mjw_step_optimized.py:2683-2742, called at :4708) and, when
taken after the call as well, its results.  With it

* a machine that has the reference installed can record golden vectors with
  ``capture`` around the reference's own ``solve_with_scratch``, and any other machine
  can replay them against this library (``load`` gives host ``Model`` / ``Data``
  stand-ins that ``solve_with_scratch`` and the CPU oracle accept);
* the fixtures under ``tests/golden`` are stored in the same format.

Layout (format ``imnewton-solver-state/1``): scalars and arrays under the prefixes
``model/``, ``in/`` (inputs of the call), ``out/`` (results, optional) and ``ctx/``
(solver context arrays after the call, optional).  Arrays keep mujoco-warp's names and
shapes; ``efc.J`` is stored with exactly ``nv`` columns.  Any array type that numpy,
torch or the ``ptr/shape/strides`` protocol of Warp arrays can express is accepted.
"""

from __future__ import annotations

from pathlib import Path
from types import SimpleNamespace
from typing import Any, Callable

import numpy as np

from . import mjw_model
from .mjw_model import Constraint, Data, Model, Option, Statistic

FORMAT = "imnewton-solver-state/1"

_MODEL_ARRAYS = (
    "dof_parentid", "M_rowadr", "M_rownnz", "M_colind", "M_hinit_i", "M_mulm_rowadr", "M_mulm_col", "M_mulm_madr",
    "body_parentid", "body_dofadr", "body_dofnum", "geom_bodyid", "nxn_geom_pair_filtered",
)
_MODEL_SCALARS = ("nv", "nv_pad", "is_sparse", "neq", "nflex", "ntendon")
_OPT_SCALARS = ("iterations", "ls_iterations", "cone", "solver", "integrator", "disableflags", "warn_overflow")
_OPT_ARRAYS = ("tolerance", "ls_tolerance", "impratio_invsqrt")
_IN_DATA = ("nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M")
_IN_EFC = ("J", "D", "aref", "frictionloss")
_OUT_DATA = ("qacc", "qfrc_constraint", "solver_niter", "overflow")
_OUT_EFC = ("force", "state", "Ma")
_CTX = (
    "Jaref", "jv", "search", "mv", "grad", "h", "hfactor", "search_dot", "grad_dot", "grad_scale", "newton_decrement",
    "improvement", "alpha", "done", "search_unchanged", "ls_exhausted", "quad_changed_ids", "quad_changed_count",
    "state_changed_count",
)


def to_numpy(a: Any) -> np.ndarray | None:
    """Host copy of a numpy array, a torch tensor, or an array that has ``numpy()``
    (Warp arrays do)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return np.array(a)
    if hasattr(a, "detach"):
        return a.detach().cpu().numpy().copy()
    if hasattr(a, "numpy"):
        return np.array(a.numpy())
    return np.asarray(a)


def _put(out: dict, key: str, a: Any) -> None:
    v = to_numpy(a)
    if v is not None:
        out[key] = v


def _model_entries(m: Any) -> dict:
    out: dict = {}
    for name in _MODEL_SCALARS:
        out[f"model/{name}"] = np.asarray(int(getattr(m, name, 0) or 0))
    for name in _MODEL_ARRAYS:
        _put(out, f"model/{name}", getattr(m, name, None))
    for name in _OPT_SCALARS:
        out[f"model/opt/{name}"] = np.asarray(int(getattr(m.opt, name, 0) or 0))
    for name in _OPT_ARRAYS:
        _put(out, f"model/opt/{name}", getattr(m.opt, name, None))
    _put(out, "model/stat/meaninertia", m.stat.meaninertia)
    return out


def _data_entries(m: Any, d: Any, prefix: str, data_fields, efc_fields) -> dict:
    out: dict = {}
    for name in data_fields:
        _put(out, f"{prefix}/{name}", getattr(d, name, None))
    for name in efc_fields:
        a = to_numpy(getattr(d.efc, name, None))
        if a is not None and name == "J":
            a = np.ascontiguousarray(a[..., : int(m.nv)])
        if a is not None:
            out[f"{prefix}/efc/{name}"] = a
    return out


def snapshot_inputs(m: Any, d: Any) -> dict:
    """The arrays a solve reads, as a dict of numpy arrays (keys as in the file)."""
    out = {"format": np.asarray(FORMAT), "in/nworld": np.asarray(int(d.nworld)), "in/njmax": np.asarray(int(d.njmax))}
    out.update(_model_entries(m))
    out.update(_data_entries(m, d, "in", _IN_DATA, _IN_EFC))
    return out


def snapshot_outputs(m: Any, d: Any, ctx: Any = None) -> dict:
    """The arrays a solve writes (and the context arrays when ``ctx`` is given)."""
    out = _data_entries(m, d, "out", _OUT_DATA, _OUT_EFC)
    if ctx is not None:
        for name in _CTX:
            _put(out, f"ctx/{name}", getattr(ctx, name, None))
    return out


def save(path: str | Path, entries: dict) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(path, **{k.replace("/", "__"): v for k, v in entries.items()})
    return path


def dump(path: str | Path, m: Any, d: Any, ctx: Any = None, *, with_outputs: bool = False) -> Path:
    """Write the solver-facing state of (m, d) to ``path``.  Call it before the solve
    for an input-only file, or after the solve with ``with_outputs=True`` when ``d``
    still holds the inputs (the solve overwrites none of them)."""
    entries = snapshot_inputs(m, d)
    if with_outputs:
        entries.update(snapshot_outputs(m, d, ctx))
    return save(path, entries)


def read(path: str | Path) -> dict:
    with np.load(Path(path), allow_pickle=False) as z:
        entries = {k.replace("__", "/"): z[k] for k in z.files}
    if str(entries.get("format")) != FORMAT:
        raise ValueError(f"{path}: not a {FORMAT} file")
    return entries


def load(path: str | Path) -> tuple[Model, Data, SimpleNamespace | None, SimpleNamespace | None]:
    """(Model, Data, outputs, ctx) on the host.  ``Data`` carries the inputs and zeroed
    result arrays; ``outputs`` (qacc, qfrc_constraint, solver_niter, overflow,
    efc_force, efc_state, efc_Ma) and ``ctx`` are None when the file holds none."""
    e = read(path)
    g = lambda k: e.get(k)  # noqa: E731
    opt = Option(
        **{n: int(e[f"model/opt/{n}"]) for n in _OPT_SCALARS},
        **{n: g(f"model/opt/{n}") for n in _OPT_ARRAYS},
    )
    nv = int(e["model/nv"])
    pack = None
    if g("model/M_mulm_col") is not None and g("model/M_mulm_madr") is not None:
        pack = mjw_model.pack_mulm(e["model/M_mulm_col"], e["model/M_mulm_madr"])
    m = Model(
        nv=nv, nv_pad=int(e["model/nv_pad"]), opt=opt, stat=Statistic(meaninertia=g("model/stat/meaninertia")),
        is_sparse=bool(int(e["model/is_sparse"])), dof_parentid=g("model/dof_parentid"),
        M_rowadr=g("model/M_rowadr"), M_rownnz=g("model/M_rownnz"), M_colind=g("model/M_colind"),
        M_hinit_i=g("model/M_hinit_i"), M_mulm_rowadr=g("model/M_mulm_rowadr"), M_mulm_col=g("model/M_mulm_col"),
        M_mulm_madr=g("model/M_mulm_madr"), M_mulm_pack=pack,
        body_parentid=g("model/body_parentid"), body_dofadr=g("model/body_dofadr"),
        body_dofnum=g("model/body_dofnum"), neq=int(e["model/neq"]), nflex=int(e["model/nflex"]),
        ntendon=int(e["model/ntendon"]), geom_bodyid=g("model/geom_bodyid"),
        nxn_geom_pair_filtered=g("model/nxn_geom_pair_filtered"),
    )
    W, R = int(e["in/nworld"]), int(e["in/njmax"])
    f = lambda *s: np.zeros(s, np.float32)  # noqa: E731
    d = Data(
        nworld=W, njmax=R, nefc=e["in/nefc"], ne=e["in/ne"], nf=e["in/nf"], qacc_smooth=e["in/qacc_smooth"],
        qacc_warmstart=e["in/qacc_warmstart"], qfrc_smooth=e["in/qfrc_smooth"], M=e["in/M"],
        qacc=f(W, nv), qfrc_constraint=f(W, nv),
        efc=Constraint(
            J=e["in/efc/J"], D=e["in/efc/D"], aref=e["in/efc/aref"], frictionloss=e["in/efc/frictionloss"],
            force=f(W, R), state=np.zeros((W, R), np.int32), Ma=f(W, nv),
        ),
        solver_niter=np.zeros(W, np.int32), overflow=np.zeros(W, np.int32),
    )
    outputs = None
    if "out/qacc" in e:
        outputs = SimpleNamespace(
            **{n: e[f"out/{n}"] for n in _OUT_DATA if f"out/{n}" in e},
            **{f"efc_{n}": e[f"out/efc/{n}"] for n in _OUT_EFC if f"out/efc/{n}" in e},
        )
    ctx = None
    if any(k.startswith("ctx/") for k in e):
        ctx = SimpleNamespace(**{n: e.get(f"ctx/{n}") for n in _CTX})
    return m, d, outputs, ctx


def capture(solve: Callable, directory: str | Path, *, prefix: str = "solve", limit: int = 8,
            sync: Callable[[], None] | None = None) -> Callable:
    """Wrap a ``solve_with_scratch``-like callable so that its first ``limit`` calls
    each leave ``<directory>/<prefix>_<n>.npz`` with inputs and results.  ``sync`` is
    called before each snapshot (e.g. ``torch.cuda.synchronize`` or
    ``wp.synchronize``); the wrapper must not be active during graph capture, since it
    copies device arrays to the host."""
    directory = Path(directory)
    state = {"n": 0}

    def wrapped(m, d, scratch, *args, **kwargs):
        record = state["n"] < limit
        if record:
            if sync:
                sync()
            entries = snapshot_inputs(m, d)
        result = solve(m, d, scratch, *args, **kwargs)
        if record:
            if sync:
                sync()
            entries.update(snapshot_outputs(m, d, getattr(scratch, "solver_context", None)))
            save(directory / f"{prefix}_{state['n']:04d}.npz", entries)
            state["n"] += 1
        return result

    wrapped.captured = state
    return wrapped
