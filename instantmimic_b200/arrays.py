"""Address / stride helpers over numpy arrays, torch tensors and Warp arrays.

The C ABI takes raw addresses, so the host layer accepts any array type that can
name its memory: numpy (host, used with the CPU oracle in tests), torch tensors
(device) and objects with Warp's ``ptr`` / ``shape`` / ``strides`` attributes,
which is how the reference's ``Model`` / ``Data`` buffers arrive.  A Warp array
differs from a torch tensor in ways that matter here: ``strides`` are in BYTES,
``dtype`` is a Warp type class without an ``itemsize``, ``is_contiguous`` is a
plain bool attribute, there is no ``data_ptr()``, ``cpu()`` or ``stride()``.
Everything in the package that touches a caller's array goes through this module.
"""

from __future__ import annotations

import ctypes
from typing import Any

import numpy as np

# Sizes of Warp's scalar types by name, for dtype objects that carry nothing else.
_NAMED_SIZES = {
    "bool": 1, "int8": 1, "uint8": 1, "int16": 2, "uint16": 2, "float16": 2,
    "int32": 4, "uint32": 4, "float32": 4, "int64": 8, "uint64": 8, "float64": 8,
    "float": 4, "int": 4,
}


def _is_torch(a: Any) -> bool:
    return hasattr(a, "data_ptr") and hasattr(a, "stride")


def addr(a: Any) -> int | None:
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if _is_torch(a):
        return int(a.data_ptr())
    if hasattr(a, "ptr"):
        return int(a.ptr) if a.ptr else None
    iface = getattr(a, "__cuda_array_interface__", None)
    if iface is not None:
        return int(iface["data"][0])
    raise TypeError(f"cannot take the address of {type(a).__name__}")


def shape(a: Any) -> tuple[int, ...]:
    return tuple(int(s) for s in a.shape)


def itemsize(a: Any) -> int:
    """Bytes per element.  Warp dtypes are classes: scalars carry the ctypes type in
    ``_type_``, vectors and matrices are ctypes arrays of it (``_length_`` elements);
    python ``float`` / ``int`` / ``bool`` stand for float32 / int32 / bool."""
    if isinstance(a, np.ndarray):
        return int(a.itemsize)
    if _is_torch(a):
        return int(a.element_size())
    dtype = getattr(a, "dtype", None)
    size = getattr(dtype, "itemsize", None)
    if isinstance(size, int) and size > 0:
        return size
    if isinstance(dtype, type) and issubclass(dtype, (ctypes.Array, ctypes.Structure, ctypes._SimpleCData)):
        return ctypes.sizeof(dtype)
    scalar = getattr(dtype, "_type_", None)
    if isinstance(scalar, type) and issubclass(scalar, ctypes._SimpleCData):
        return ctypes.sizeof(scalar) * int(getattr(dtype, "_length_", 1) or 1)
    name = getattr(dtype, "__name__", None) or str(dtype)
    if name in _NAMED_SIZES:
        return _NAMED_SIZES[name]
    raise TypeError(f"cannot tell the element size of dtype {dtype!r}")


def elem_strides(a: Any) -> tuple[int, ...]:
    """Strides in elements."""
    if isinstance(a, np.ndarray):
        return tuple(int(s // a.itemsize) for s in a.strides)
    if _is_torch(a):
        return tuple(int(s) for s in a.stride())
    size = itemsize(a)
    out = []
    for s in a.strides:
        if int(s) % size:
            raise ValueError(f"byte stride {int(s)} is not a multiple of the element size {size}")
        out.append(int(s) // size)
    return tuple(out)


def is_contiguous(a: Any) -> bool:
    """Row-major without gaps.  ``is_contiguous`` is a method on torch tensors and a
    bool attribute on Warp arrays."""
    if isinstance(a, np.ndarray):
        return bool(a.flags["C_CONTIGUOUS"])
    flag = getattr(a, "is_contiguous", None)
    if callable(flag):
        return bool(flag())
    if flag is not None:
        return bool(flag)
    expect, st, sh = 1, elem_strides(a), shape(a)
    for n, s in zip(reversed(sh), reversed(st)):
        if n != 1 and s != expect:
            return False
        expect *= n
    return True


def is_device(a: Any) -> bool:
    if isinstance(a, np.ndarray):
        return False
    if hasattr(a, "is_cuda") and not callable(a.is_cuda):
        return bool(a.is_cuda)
    device = getattr(a, "device", None)
    return bool(getattr(device, "is_cuda", False))


def length(a: Any) -> int:
    return int(a.shape[0])


def to_host(a: Any) -> np.ndarray:
    """Host numpy copy (or the array itself for numpy input)."""
    if isinstance(a, np.ndarray):
        return a
    if hasattr(a, "detach"):
        return a.detach().cpu().numpy()
    if hasattr(a, "numpy"):
        return np.asarray(a.numpy())
    return np.asarray(a)


_TABLES: dict = {}


def table_to_host(a: Any) -> np.ndarray:
    """Host copy of a constant model table, read from the device once per buffer: a copy
    in every call would synchronise the stream and cannot be captured in a CUDA graph.
    Only for arrays whose contents never change after model set-up."""
    if isinstance(a, np.ndarray):
        return a
    key = (addr(a), tuple(shape(a)))
    hit = _TABLES.get(key)
    if hit is None:
        if len(_TABLES) > 256:
            _TABLES.clear()
        hit = _TABLES[key] = np.array(to_host(a), copy=True)
    return hit


def as_torch(a: Any):
    """Zero-copy torch view of a caller's array (device arrays through
    ``__cuda_array_interface__``, which Warp arrays provide)."""
    import torch

    if isinstance(a, torch.Tensor):
        return a
    if isinstance(a, np.ndarray):
        return torch.from_numpy(a)
    if getattr(a, "__cuda_array_interface__", None) is not None:
        return torch.as_tensor(a, device="cuda")
    if getattr(a, "__array_interface__", None) is not None:
        return torch.from_numpy(np.asarray(a))
    raise TypeError(f"cannot view {type(a).__name__} as a torch tensor")


def device_of(a: Any):
    """torch.device of a caller's device array."""
    import torch

    if isinstance(a, torch.Tensor):
        return a.device
    device = getattr(a, "device", None)
    ordinal = getattr(device, "ordinal", None)
    if ordinal is not None:
        return torch.device("cuda", int(ordinal))
    return as_torch(a).device
