"""Solving batches whose inputs live in pinned host memory.

The reference keeps every solver buffer on the GPU, so this module has no
counterpart there; it is the public entry for callers on the other side of PCIe (a
CPU-side constraint producer, a replay of recorded solver states) and the path the
benchmark's end-to-end figure is measured through.

What it does per batch, all on one stream per slot and with nothing allocated after
construction:

* host -> device copies of the inputs.  ``efc.J`` is 78 % of a humanoid batch and the
  solver never reads rows at or beyond a world's ``nefc``.  Three ways to move it:
  ``"compact"`` (default) keeps J on the host as the ``nefc`` rows of each world back to
  back, as MuJoCo C stores ``mjData.efc_J``, copies that one contiguous block and tells
  the kernel where each world starts (``ImnData.J_world_offset``); ``"rows"`` keeps the
  padded layout and copies rows ``[0, max nefc of the chunk)`` of chunks of worlds
  with strided copies (``imn_copy_rows`` = ``cudaMemcpy2DAsync``; tight when the caller
  groups its worlds by row count, slower per byte than a contiguous copy);
  ``"whole"`` copies the padded array.  The per-row vectors (D, aref, frictionloss) are
  copied whole: their per-world segments are a few hundred bytes.
* ``solve_with_scratch`` on the device buffers.
* device -> host copies of the results (whole arrays).

Slots are independent (own device buffers, stream and pinned result buffers), so the
copies of one batch overlap the solve of another.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any

import numpy as np

from . import _lib, mjw_model
from . import mjw_step_optimized as runtime

_IN_DOF = ("qacc_smooth", "qacc_warmstart", "qfrc_smooth")
_IN_ROW = ("D", "aref", "frictionloss")
_OUT_DOF = ("qacc", "qfrc_constraint")
_OUT_ROW = ("force", "state")


@dataclass
class HostBatch:
    """Pinned host tensors of one batch plus the row count each chunk of worlds needs."""

    tensors: dict  # name -> pinned torch tensor ("efc.J" style names for row arrays)
    chunk_rows: list  # (first world, worlds, rows to copy) per chunk
    nworld: int

    def h2d_bytes(self, nv: int, ldj: int, nM: int, njmax: int, mode: str = "compact") -> int:
        total = self.nworld * 4 * (3 + 3 * nv + nM + 3 * njmax)
        if mode == "whole":
            return total + self.nworld * njmax * ldj * 4
        if mode == "rows":
            return total + sum(n * rows * 4 * ldj for _, n, rows in self.chunk_rows)
        return total + int(self.tensors["Jc"].numel()) * 4 + 8 * self.nworld

    def d2h_bytes(self, nv: int, njmax: int) -> int:
        return self.nworld * 4 * (3 * nv + 2 + 2 * njmax)


def pin_batch(d: Any, chunk: int = 256) -> HostBatch:
    """Pinned copies of a host ``Data``'s solver inputs.  ``chunk`` worlds share one
    strided copy; the rows copied for a chunk are its largest ``nefc``."""
    import torch

    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()  # noqa: E731
    t = {n: pin(getattr(d, n)) for n in ("nefc", "ne", "nf", "M") + _IN_DOF}
    t["J"] = pin(d.efc.J)
    compact = mjw_model.compact_jacobian(d)
    t["Jc"], t["Joff"] = pin(compact.efc.J), pin(compact.efc.J_world_offset)
    for n in _IN_ROW:
        t[n] = pin(getattr(d.efc, n))
    nefc = np.minimum(np.asarray(d.nefc), d.njmax)
    chunks = []
    for lo in range(0, d.nworld, chunk):
        hi = min(lo + chunk, d.nworld)
        chunks.append((lo, hi - lo, int(nefc[lo:hi].max()) if hi > lo else 0))
    return HostBatch(tensors=t, chunk_rows=chunks, nworld=int(d.nworld))


def group_by_row_count(d: Any):
    """A copy of host ``Data`` with its worlds reordered by descending ``nefc`` (what a
    producer that buckets its worlds hands over), and the permutation used."""
    order = np.argsort(-np.asarray(d.nefc), kind="stable")
    out = mjw_model.slice_worlds(d, 0, d.nworld)
    for name in ("nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M", "qacc",
                 "qfrc_constraint", "solver_niter", "overflow"):
        setattr(out, name, np.ascontiguousarray(getattr(d, name)[order]))
    for name in ("J", "D", "aref", "frictionloss", "force", "state", "Ma"):
        setattr(out.efc, name, np.ascontiguousarray(getattr(d.efc, name)[order]))
    return out, order


class HostBatchPipeline:
    """``slots`` independent (device buffers, stream, pinned results) sets for batches of
    one shape.  ``submit`` enqueues copies + solve + copies and returns at once;
    ``result`` waits for that slot and returns its pinned result tensors."""

    def __init__(self, m_dev: Any, template: Any, device: Any, *, slots: int = 2, sparse_groups=None,
                 mode: str = "compact"):
        import torch

        if mode not in ("compact", "rows", "whole"):
            raise ValueError("mode must be compact, rows or whole")
        self.m = m_dev
        self.mode = mode
        self.device = device
        self.slots = []
        for _ in range(slots):
            dd = mjw_model.to_device(mjw_model.make_data(_host_model_view(m_dev), template.nworld, template.njmax),
                                     device)
            if mode == "compact":
                # the same storage as (all rows, nv); every submit says where worlds start
                dd.efc.J = dd.efc.J.view(template.nworld * template.njmax, -1)
                dd.efc.J_world_offset = torch.zeros(template.nworld, dtype=torch.int64, device=device)
            sc = runtime.make_optimized_fwd_position_scratch(m_dev, dd, device)
            if sparse_groups is not None:
                runtime.refresh_sparse_hessian(m_dev, dd, sc, sparse_groups, device)
            pin = lambda t: torch.empty(t.shape, dtype=t.dtype).pin_memory()  # noqa: E731
            out = {n: pin(getattr(dd, n)) for n in _OUT_DOF + ("solver_niter", "overflow")}
            out["Ma"] = pin(dd.efc.Ma)
            for n in _OUT_ROW:
                out[n] = pin(getattr(dd.efc, n))
            self.slots.append({"dd": dd, "sc": sc, "stream": torch.cuda.Stream(device=device),
                               "done": torch.cuda.Event(), "out": out, "batch": None})
        self.lib = _lib.lib()

    def _rows(self, dst, src, lo, n, rows, to_host, stream):
        """Rows [0, rows) of worlds [lo, lo + n) of a (W, R, ...) array pair."""
        pitch = dst.stride(0) * dst.element_size()
        width = rows * dst.stride(1) * dst.element_size()
        off = lo * pitch
        rc = self.lib.imn_copy_rows(dst.data_ptr() + off, pitch, src.data_ptr() + off, pitch, width, n,
                                    1 if to_host else 0, stream)
        _lib.check(rc, "imn_copy_rows")

    def submit(self, k: int, batch: HostBatch) -> None:
        import torch

        sl = self.slots[k % len(self.slots)]
        dd, t = sl["dd"], batch.tensors
        handle = int(sl["stream"].cuda_stream)
        with torch.cuda.stream(sl["stream"]):
            for n in ("nefc", "ne", "nf", "M") + _IN_DOF:
                getattr(dd, n).copy_(t[n], non_blocking=True)
            for name in _IN_ROW:
                getattr(dd.efc, name).copy_(t[name], non_blocking=True)
            if self.mode == "compact":
                dd.efc.J[: t["Jc"].shape[0]].copy_(t["Jc"], non_blocking=True)
                dd.efc.J_world_offset.copy_(t["Joff"], non_blocking=True)
            elif self.mode == "rows":
                for lo, n, rows in batch.chunk_rows:
                    if rows:
                        self._rows(dd.efc.J, t["J"], lo, n, rows, False, handle)
            else:
                dd.efc.J.copy_(t["J"], non_blocking=True)
            runtime.solve_with_scratch(self.m, dd, sl["sc"], use_optimized_kernel=True, stream=sl["stream"])
            out = sl["out"]
            for n in _OUT_DOF + ("solver_niter", "overflow"):
                out[n].copy_(getattr(dd, n), non_blocking=True)
            out["Ma"].copy_(dd.efc.Ma, non_blocking=True)
            for name in _OUT_ROW:
                out[name].copy_(getattr(dd.efc, name), non_blocking=True)
            sl["done"].record(sl["stream"])
        sl["batch"] = batch

    def result(self, k: int) -> dict:
        sl = self.slots[k % len(self.slots)]
        sl["done"].synchronize()
        return sl["out"]


def _host_model_view(m_dev: Any):
    """``make_data`` only needs nv and nM of the model."""
    from types import SimpleNamespace

    return SimpleNamespace(nv=int(m_dev.nv), nM=int(m_dev.M_colind.shape[0]))
