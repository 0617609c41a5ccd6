"""Address / stride helpers over numpy arrays, torch tensors and Warp arrays.

The C ABI takes raw addresses, so the host layer accepts any array type that can
name its memory: numpy (host, used with the CPU oracle in tests), torch tensors
(device) and objects with Warp's ``ptr`` / ``shape`` / ``strides`` attributes,
which is how the reference's ``Model`` / ``Data`` buffers arrive.
"""

from __future__ import annotations

from typing import Any

import numpy as np


def addr(a: Any) -> int | None:
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        return int(a.data_ptr())
    if hasattr(a, "ptr"):
        return int(a.ptr) if a.ptr else None
    iface = getattr(a, "__cuda_array_interface__", None)
    if iface is not None:
        return int(iface["data"][0])
    raise TypeError(f"cannot take the address of {type(a).__name__}")


def shape(a: Any) -> tuple[int, ...]:
    return tuple(int(s) for s in a.shape)


def elem_strides(a: Any) -> tuple[int, ...]:
    """Strides in elements."""
    if isinstance(a, np.ndarray):
        return tuple(int(s // a.itemsize) for s in a.strides)
    if hasattr(a, "data_ptr"):
        return tuple(int(s) for s in a.stride())
    itemsize = 4
    dtype = getattr(a, "dtype", None)
    size = getattr(dtype, "itemsize", None)
    if isinstance(size, int) and size > 0:
        itemsize = size
    return tuple(int(s // itemsize) for s in a.strides)


def is_device(a: Any) -> bool:
    if isinstance(a, np.ndarray):
        return False
    if hasattr(a, "is_cuda"):
        return bool(a.is_cuda)
    device = getattr(a, "device", None)
    return bool(getattr(device, "is_cuda", False))


def length(a: Any) -> int:
    return int(a.shape[0])
