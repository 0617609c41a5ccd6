"""A stand-in for ``warp.array`` with the attributes the reference's Model / Data /
solver-context buffers have, over memory owned by a torch tensor.  It deliberately
offers nothing torch-like: no ``data_ptr()``, ``stride()``, ``cpu()`` or ``device.type``;
``strides`` are bytes, ``dtype`` is a class without ``itemsize``, ``is_contiguous`` is a
bool attribute.  Code that handles these objects handles live Warp arrays."""

from __future__ import annotations

import ctypes
from dataclasses import fields, is_dataclass, replace
from types import SimpleNamespace

import numpy as np


class float32:  # noqa: N801 - Warp's scalar types are lower-case classes
    _type_ = ctypes.c_float


class int32:  # noqa: N801
    _type_ = ctypes.c_int32


class uint8:  # noqa: N801
    _type_ = ctypes.c_uint8


class bool_:  # noqa: N801 - Warp's bool: one byte
    _type_ = ctypes.c_bool
    __name__ = "bool"


class uint32:  # noqa: N801
    _type_ = ctypes.c_uint32


_DTYPES = {"float32": float32, "int32": int32, "uint8": uint8, "bool": bool_, "uint32": uint32}


class _Device:
    def __init__(self, cuda: bool, ordinal: int):
        self.is_cuda = cuda
        self.ordinal = ordinal if cuda else None
        self.alias = f"cuda:{ordinal}" if cuda else "cpu"


class FakeWarpArray:
    def __init__(self, tensor, dtype=None):
        import torch

        self._t = tensor  # keeps the memory alive
        self.ptr = int(tensor.data_ptr())
        self.shape = tuple(int(s) for s in tensor.shape)
        self.strides = tuple(int(s) * tensor.element_size() for s in tensor.stride())
        self.ndim = tensor.dim()
        self.size = int(tensor.numel())
        name = str(tensor.dtype).replace("torch.", "")
        self.dtype = dtype if dtype is not None else _DTYPES[name]
        self.is_contiguous = bool(tensor.is_contiguous())
        self.device = _Device(tensor.is_cuda, tensor.device.index or 0)
        assert isinstance(tensor, torch.Tensor)

    def zero_(self):
        self._t.zero_()

    def fill_(self, v):
        self._t.fill_(v)

    def numpy(self):
        return self._t.detach().cpu().numpy()

    @property
    def __cuda_array_interface__(self):
        if not self.device.is_cuda:
            raise AttributeError("__cuda_array_interface__")
        return self._t.__cuda_array_interface__

    @property
    def __array_interface__(self):
        if self.device.is_cuda:
            raise AttributeError("__array_interface__")
        return self._t.numpy().__array_interface__


def wrap(obj):
    """Copy of a (nested) Model / Data / context container with every torch tensor or
    numpy array replaced by a FakeWarpArray over the same memory."""
    import torch

    if isinstance(obj, np.ndarray):
        return FakeWarpArray(torch.from_numpy(obj))
    if isinstance(obj, torch.Tensor):
        return FakeWarpArray(obj)
    if is_dataclass(obj) and not isinstance(obj, type):
        return replace(obj, **{f.name: wrap(getattr(obj, f.name)) for f in fields(obj)})
    if isinstance(obj, SimpleNamespace):
        return SimpleNamespace(**{k: wrap(v) for k, v in vars(obj).items()})
    if hasattr(obj, "__dict__") and type(obj).__name__ == "SolverContext":
        out = SimpleNamespace()
        for k, v in vars(obj).items():
            setattr(out, k, wrap(v) if isinstance(v, (torch.Tensor, np.ndarray)) else v)
        return out
    return obj
