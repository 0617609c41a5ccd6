"""``torch.library`` registration of the solve: ``torch.ops.imnewton.solve``.

For callers that live in torch (the reference aligns its Warp stream with a torch
stream and hands torch views of the Warp buffers around,
src/instantmimic/envs/direct_rl_env.py:898-913): the op takes the Data and context
buffers as tensors, declares which ones it writes, and launches on torch's current
stream, so it composes with CUDA-graph capture and is opaque to ``torch.compile``.
The model and its options are registered once and passed as an integer handle; the
tensors are handed to the C ABI as raw pointers, nothing is copied.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import Any, Sequence

import torch

from . import mjw_step_optimized as runtime
from .mjw_model import Constraint

_MODELS: dict[int, tuple[Any, Any]] = {}

# positions in the tensor lists of the op
INPUTS = ("nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M", "efc_J", "efc_D", "efc_aref",
          "efc_frictionloss")
OUTPUTS = ("qacc", "qfrc_constraint", "efc_Ma", "efc_force", "efc_state", "solver_niter", "overflow")


def register_model(m: Any, scratch: Any) -> int:
    """Remember a (Model, scratch) pair; returns the handle the op takes."""
    handle = len(_MODELS) + 1
    _MODELS[handle] = (m, scratch)
    return handle


@torch.library.custom_op("imnewton::solve", mutates_args=("outputs",), device_types="cuda")
def solve(model: int, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor]) -> None:
    """One Newton constraint solve of every world (``solve_with_scratch``)."""
    m, scratch = _MODELS[model]
    i = dict(zip(INPUTS, inputs))
    o = dict(zip(OUTPUTS, outputs))
    d = SimpleNamespace(
        nworld=int(i["nefc"].shape[0]), njmax=int(i["efc_D"].shape[1]),
        nefc=i["nefc"], ne=i["ne"], nf=i["nf"], qacc_smooth=i["qacc_smooth"], qacc_warmstart=i["qacc_warmstart"],
        qfrc_smooth=i["qfrc_smooth"], M=i["M"], qacc=o["qacc"], qfrc_constraint=o["qfrc_constraint"],
        solver_niter=o["solver_niter"], overflow=o["overflow"],
        efc=Constraint(J=i["efc_J"], D=i["efc_D"], aref=i["efc_aref"], frictionloss=i["efc_frictionloss"],
                       force=o["efc_force"], state=o["efc_state"], Ma=o["efc_Ma"]),
    )
    runtime.solve_with_scratch(m, d, scratch, use_optimized_kernel=True)


@solve.register_fake
def _(model, inputs, outputs):
    return None


def solve_data(model: int, d: Any) -> None:
    """``torch.ops.imnewton.solve`` on the buffers of a Data container."""
    ins = [getattr(d, n) if not n.startswith("efc_") else getattr(d.efc, n[4:]) for n in INPUTS]
    outs = [getattr(d, n) if not n.startswith("efc_") else getattr(d.efc, n[4:]) for n in OUTPUTS]
    torch.ops.imnewton.solve(model, ins, outs)
