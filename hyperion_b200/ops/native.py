"""Glue between torch tensors and the exported C launchers of ``csrc``.

Every launcher takes raw device pointers, sizes and the CUDA stream and returns an int: 0 on
success, a positive ``cudaError_t`` if the launch failed, a negative code if it refused its
arguments.  Nothing here falls back to another implementation: a tensor that is not on a CUDA
device, a failed build or a refused size raises.
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch

from ..csrc import build

_REFUSALS = {-1: "bad argument", -2: "unsupported size", -3: "scratch too small", -4: "set-up failed"}


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed."""


def ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    if tensor is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(tensor.data_ptr())


_bound_stream: list = [None]  # the stream a step has bound for its launches, or None


def stream_ptr() -> ctypes.c_void_p:
    """The stream launches go to: the one bound by ``stream_bound`` if any, else torch's current stream."""
    bound = _bound_stream[0]
    return bound if bound is not None else ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_bound:
    """``with stream_bound():`` looks torch's current stream up once; the launches inside use it without asking again.
    Nesting rebinds (a graph capture inside a step launches on the capture's stream)."""

    def __enter__(self):
        self.previous = _bound_stream[0]
        _bound_stream[0] = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        _bound_stream[0] = self.previous
        return False


def require_cuda(*tensors: torch.Tensor | None) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("the kernels run on a CUDA device only; got a tensor on " + str(tensor.device))


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (the current one by default), asked once per device: grids and split counts follow it."""
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    found = _sm_counts.get(index)
    if found is None:
        found = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return found


LAUNCHES = [0]  # launcher calls that succeeded, for reports of how much of a step is this package's own code


def check(code: int, what: str) -> None:
    if code == 0:
        LAUNCHES[0] += 1
        return
    if code < 0:
        raise KernelError(f"{what}: launcher refused its arguments ({_REFUSALS.get(code, code)})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def is_bf16(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.bfloat16:
        return 1
    if tensor.dtype == torch.float32:
        return 0
    raise KernelError(f"unsupported element type {tensor.dtype} (float32 and bfloat16 only)")


_libraries: dict = {}


def library(module: str, **defines: Any) -> ctypes.CDLL:
    key = (module, tuple(sorted(defines.items()))) if defines else module
    found = _libraries.get(key)
    if found is None:
        found = _libraries[key] = build.load(module, defines)
    return found


i32 = int  # a Python int is passed as a C int by ctypes itself; the name marks which arguments are 32-bit


def f32(value: float) -> ctypes.c_float:
    return ctypes.c_float(float(value))
