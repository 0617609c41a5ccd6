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
  ``"whole"`` copies the padded array; ``"sparse"`` keeps the rows on the host as values +
  column indices + row starts (what MuJoCo C holds with ``jacobian="sparse"``: ``efc_J``,
  ``efc_J_colind``, ``efc_J_rowadr``), copies those and writes the dense rows on the device
  (``imn_expand_rows``), so that only the nonzeros cross PCIe; ``"sparse8"`` is the same with
  the column indices as bytes (a fused-path model has at most 79 dofs): 5 instead of 8 bytes
  per nonzero, for producers that emit their rows in this form.  The per-row vectors (D, aref, frictionloss) are copied whole: their
  per-world segments are a few hundred bytes.
* ``solve_with_scratch`` on the device buffers.
* device -> host copies of the results (whole arrays).

Slots are independent (own device buffers, stream and pinned result buffers), so the
copies of one batch overlap the solve of another.  A slot's chain is copy in -> solve ->
copy out, so two slots keep the PCIe link busy only while the copy in is at least as long
as solve + copy out; with the sparse modes (copy in about as long as the solve) take three.
The sparse modes also move every input in ONE pinned buffer and every result in another
(the device arrays are views of two device buffers): one copy each way per batch.
"""

from __future__ import annotations

import ctypes as C
import os
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
        if mode in ("sparse", "sparse8"):
            return int(self.tensors["packed_meta" if mode == "sparse" else "packed8_meta"][5])  # the one buffer copied
        return total + int(self.tensors["Jc"].numel()) * 4 + 8 * self.nworld

    def d2h_bytes(self, nv: int, njmax: int, mode: str = "compact") -> int:
        if mode in ("sparse", "sparse8"):
            return result_layout(self.nworld, njmax, nv)[1]
        return self.nworld * 4 * (3 * nv + 2 + 2 * njmax)


_ALIGN = 256


def _up(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


def packed_layout(nworld: int, njmax: int, nv: int, nM: int) -> tuple[dict, int]:
    """Byte offsets of the fixed-size inputs inside one packed transfer buffer (each
    segment starts on a 256-byte boundary) and the offset where the batch-dependent part
    begins: row starts, values and column indices of the sparse rows, then D, aref and
    frictionloss of the live rows."""
    W, R = nworld, njmax
    fixed = [("nefc", "int32", (W,)), ("ne", "int32", (W,)), ("nf", "int32", (W,)), ("Joff", "int64", (W,)),
             ("M", "float32", (W, nM)), ("qacc_smooth", "float32", (W, nv)), ("qacc_warmstart", "float32", (W, nv)),
             ("qfrc_smooth", "float32", (W, nv))]
    del R  # the per-row inputs travel compacted, in the batch-dependent part
    offsets, o = {}, 0
    for name, dtype, shape in fixed:
        offsets[name] = (o, dtype, shape)
        o += _up(int(np.prod(shape)) * np.dtype(dtype).itemsize)
    return offsets, o


def result_layout(nworld: int, njmax: int, nv: int) -> tuple[dict, int]:
    """The same for the results that go back in one transfer."""
    W, R = nworld, njmax
    out = [("qacc", "float32", (W, nv)), ("qfrc_constraint", "float32", (W, nv)), ("Ma", "float32", (W, nv)),
           ("solver_niter", "int32", (W,)), ("overflow", "int32", (W,)), ("force", "float32", (W, R)),
           ("state", "int32", (W, R))]
    offsets, o = {}, 0
    for name, dtype, shape in out:
        offsets[name] = (o, dtype, shape)
        o += _up(int(np.prod(shape)) * np.dtype(dtype).itemsize)
    return offsets, o


def _views(buffer, offsets: dict) -> dict:
    """Typed tensor views of a uint8 torch buffer at the layout's offsets."""
    import torch

    out = {}
    for name, (o, dtype, shape) in offsets.items():
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        out[name] = buffer[o:o + n].view(getattr(torch, dtype)).view(shape)
    return out


def pin_batch(d: Any, chunk: int = 256) -> HostBatch:
    """Pinned copies of a host ``Data``'s solver inputs.  ``chunk`` worlds share one
    strided copy; the rows copied for a chunk are its largest ``nefc``."""
    import torch

    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()  # noqa: E731
    t = {n: pin(getattr(d, n)) for n in ("nefc", "ne", "nf", "M") + _IN_DOF}
    t["J"] = pin(d.efc.J)
    compact = mjw_model.compact_jacobian(d)
    t["Jc"], t["Joff"] = pin(compact.efc.J), pin(compact.efc.J_world_offset)
    # the same rows as values + column indices + row starts; an entry is kept when any bit
    # of it is set, so that a stored -0.0 comes back as -0.0
    rows = np.ascontiguousarray(compact.efc.J, np.float32)
    keep = rows.view(np.uint32) != 0
    if int(nefc_total(d)) == 0:
        keep[:] = False
    t["Jval"] = pin(rows[keep])
    t["Jcol"] = pin(np.nonzero(keep)[1].astype(np.int32))
    if rows.shape[1] <= 256:
        t["Jcol8"] = pin(np.nonzero(keep)[1].astype(np.uint8))
    t["Jadr"] = pin(np.concatenate(([0], np.cumsum(keep.sum(axis=1)))).astype(np.int32))
    for n in _IN_ROW:
        t[n] = pin(getattr(d.efc, n))
    nefc = np.minimum(np.asarray(d.nefc), d.njmax)
    chunks = []
    for lo in range(0, d.nworld, chunk):
        hi = min(lo + chunk, d.nworld)
        chunks.append((lo, hi - lo, int(nefc[lo:hi].max()) if hi > lo else 0))
    # everything a sparse-row submit moves, in ONE pinned buffer (one host -> device copy);
    # D, aref and frictionloss as the values of the live rows, in the compact Jacobian's order
    live = np.arange(d.njmax)[None, :] < nefc[:, None]
    live_rows = {name: np.ascontiguousarray(np.asarray(getattr(d.efc, name), np.float32)[live]) for name in _IN_ROW}
    if rows.shape[0] != int(live.sum()):  # a batch without any row carries one dummy row
        live_rows = {name: np.zeros(rows.shape[0], np.float32) for name in _IN_ROW}
    nv, nM = int(d.efc.J.shape[-1]), int(d.M.shape[1])
    offsets, var0 = packed_layout(int(d.nworld), int(d.njmax), nv, nM)
    for key, col in (("packed", "Jcol"), ("packed8", "Jcol8")):
        if col not in t:
            continue
        nadr, nnz = int(t["Jadr"].numel()), int(t["Jval"].numel())
        nrows = nadr - 1
        adr_off = var0
        val_off = adr_off + _up(4 * nadr)
        col_off = val_off + _up(4 * nnz)
        vec_off = col_off + _up(int(t[col].element_size()) * nnz)  # D | aref | frictionloss, nrows each
        used = vec_off + 3 * _up(4 * nrows)
        buf = torch.zeros(used, dtype=torch.uint8).pin_memory()
        views = _views(buf, offsets)
        for name in views:
            views[name].copy_(t[name])
        buf[adr_off:adr_off + 4 * nadr].view(torch.int32).copy_(t["Jadr"])
        buf[val_off:val_off + 4 * nnz].view(torch.float32).copy_(t["Jval"])
        buf[col_off:col_off + int(t[col].element_size()) * nnz].view(t[col].dtype).copy_(t[col])
        for i, name in enumerate(_IN_ROW):
            o = vec_off + i * _up(4 * nrows)
            buf[o:o + 4 * nrows].view(torch.float32).copy_(torch.from_numpy(live_rows[name]))
        t[key] = buf
        t[key + "_meta"] = (adr_off, val_off, col_off, nadr, nnz, used, vec_off, _up(4 * nrows))
    return HostBatch(tensors=t, chunk_rows=chunks, nworld=int(d.nworld))


def nefc_total(d: Any) -> int:
    return int(np.minimum(np.asarray(d.nefc), d.njmax).sum())


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

        if mode not in ("compact", "rows", "whole", "sparse", "sparse8"):
            raise ValueError("mode must be compact, rows, whole, sparse or sparse8")
        self.m = m_dev
        self.mode = mode
        self.device = device
        self.slots = []
        for _ in range(slots):
            dd = mjw_model.to_device(mjw_model.make_data(_host_model_view(m_dev), template.nworld, template.njmax),
                                     device)
            sparse = None
            if mode in ("compact", "sparse", "sparse8"):
                # the same storage as (all rows, nv); every submit says where worlds start
                dd.efc.J = dd.efc.J.view(template.nworld * template.njmax, -1)
                dd.efc.J_world_offset = torch.zeros(template.nworld, dtype=torch.int64, device=device)
            outdev = None
            if mode in ("sparse", "sparse8"):
                # the inputs are views of ONE device buffer that a submit fills with one copy, the
                # results views of another that goes back with one copy
                W, R, nv, nM = template.nworld, template.njmax, int(m_dev.nv), int(m_dev.M_colind.shape[0])
                offsets, var0 = packed_layout(W, R, nv, nM)
                cb = 4 if mode == "sparse" else 1
                cap = var0 + _up(4 * (W * R + 1)) + _up(4 * W * R * nv) + _up(cb * W * R * nv) + 3 * _up(4 * W * R)
                inbuf = torch.zeros(cap, dtype=torch.uint8, device=device)
                v = _views(inbuf, offsets)
                for n in ("nefc", "ne", "nf", "M") + _IN_DOF:
                    setattr(dd, n, v[n])
                dd.efc.J_world_offset = v["Joff"]
                roff, rbytes = result_layout(W, R, nv)
                outdev = torch.zeros(rbytes, dtype=torch.uint8, device=device)
                rv = _views(outdev, roff)
                for n in _OUT_DOF + ("solver_niter", "overflow"):
                    setattr(dd, n, rv[n])
                dd.efc.Ma, dd.efc.force, dd.efc.state = rv["Ma"], rv["force"], rv["state"]
                sparse = {"in": inbuf, "colbytes": cb, "roff": roff}
            sc = runtime.make_optimized_fwd_position_scratch(m_dev, dd, device)
            if sparse_groups is not None:
                runtime.refresh_sparse_hessian(m_dev, dd, sc, sparse_groups, device)
            pin = lambda t: torch.empty(t.shape, dtype=t.dtype).pin_memory()  # noqa: E731
            if outdev is not None:
                sparse["outdev"] = outdev
                sparse["outpin"] = torch.zeros(outdev.numel(), dtype=torch.uint8).pin_memory()
                out = _views(sparse["outpin"], sparse["roff"])
            else:
                out = {n: pin(getattr(dd, n)) for n in _OUT_DOF + ("solver_niter", "overflow")}
                out["Ma"] = pin(dd.efc.Ma)
                for n in _OUT_ROW:
                    out[n] = pin(getattr(dd.efc, n))
            self.slots.append({"dd": dd, "sc": sc, "stream": torch.cuda.Stream(device=device),
                               "done": torch.cuda.Event(), "out": out, "batch": None, "sparse": sparse})
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
            if self.mode in ("sparse", "sparse8"):
                sp = sl["sparse"]
                key = "packed" if self.mode == "sparse" else "packed8"
                adr_off, val_off, col_off, nadr, _, used, vec_off, vec_step = t[key + "_meta"]
                sp["in"][:used].copy_(t[key], non_blocking=True)
                base = sp["in"].data_ptr()
                rc = self.lib.imn_expand_row_vectors(
                    base + vec_off, base + vec_off + vec_step, base + vec_off + 2 * vec_step,
                    dd.efc.J_world_offset.data_ptr(), int(dd.efc.J.stride(0)), dd.nefc.data_ptr(), int(dd.njmax),
                    dd.efc.D.data_ptr(), dd.efc.aref.data_ptr(), dd.efc.frictionloss.data_ptr(),
                    int(dd.efc.D.stride(0)), int(dd.nworld), handle)
                _lib.check(rc, "imn_expand_row_vectors")
                rc = self.lib.imn_expand_rows(base + val_off, base + col_off, sp["colbytes"], base + adr_off, nadr - 1,
                                              int(self.m.nv), dd.efc.J.data_ptr(), int(dd.efc.J.stride(0)), handle)
                _lib.check(rc, "imn_expand_rows")
                runtime.solve_with_scratch(self.m, dd, sl["sc"], use_optimized_kernel=True, stream=sl["stream"])
                sp["outpin"].copy_(sp["outdev"], non_blocking=True)
                sl["done"].record(sl["stream"])
                sl["batch"] = batch
                return
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


def _cpu_list(text: str) -> set[int]:
    """CPUs of a sysfs ``cpulist`` ("0-31,64-95")."""
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if part:
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


class host_near_device:
    """Context manager: run the calling thread on the CPUs of the NUMA node the GPU hangs
    off, so that pinned buffers allocated inside (``pin_batch``, ``HostBatchPipeline``) are
    first touched, hence placed, in that node's memory.  With one process per GPU on a
    two-socket host the host-to-device copies of all ranks otherwise read one socket's
    memory.  Does nothing (``node`` stays None) when the platform does not say which node
    the device belongs to.  The previous affinity is restored on exit.

    ``pci_bus_id`` is the device's "domain:bus:device.function" address; by default it is
    asked of torch for CUDA device ``device_index``.
    """

    def __init__(self, device_index: int = 0, *, pci_bus_id: str | None = None, sysfs: str = "/sys"):
        self.device_index, self.pci_bus_id, self.sysfs = device_index, pci_bus_id, sysfs
        self.node: int | None = None
        self._saved: set[int] | None = None

    def _address(self) -> str | None:
        if self.pci_bus_id is not None:
            return self.pci_bus_id.lower()
        try:
            import torch

            p = torch.cuda.get_device_properties(self.device_index)
            return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        except Exception:  # no CUDA device, or a torch without the PCI fields
            return None

    def __enter__(self):
        address = self._address()
        if address is None or not hasattr(os, "sched_setaffinity"):
            return self
        try:
            with open(os.path.join(self.sysfs, "bus/pci/devices", address, "numa_node")) as f:
                node = int(f.read())
            if node < 0:
                return self
            with open(os.path.join(self.sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
                cpus = _cpu_list(f.read()) & os.sched_getaffinity(0)
            if not cpus:
                return self
            self._saved = os.sched_getaffinity(0)
            os.sched_setaffinity(0, cpus)
            self.node = node
        except (OSError, ValueError):
            self._saved = None
        return self

    def __exit__(self, *exc):
        if self._saved is not None:
            os.sched_setaffinity(0, self._saved)
            self._saved = None
        return False


def _host_model_view(m_dev: Any):
    """``make_data`` only needs nv and nM of the model."""
    from types import SimpleNamespace

    return SimpleNamespace(nv=int(m_dev.nv), nM=int(m_dev.M_colind.shape[0]))
