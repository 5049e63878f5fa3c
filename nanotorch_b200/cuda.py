"""CUDA device handling: the reference's ``nanotorch.cuda`` module (src/nanotorch/cuda.py:1-33)."""

from typing import Literal

from . import _C
from .tensor import std_device

Device = _C.Device
DeviceLiteral = Literal["cpu", "cuda"]


def is_available() -> bool:
    """True when a CUDA device is usable."""
    return _C.is_cuda_available()


def sync() -> None:
    """Wait for every kernel enqueued on the library's stream."""
    _C.cuda_sync()


def get_std_device(device) -> Device:
    """"cpu" / "cuda" / Device -> Device; ValueError for anything else."""
    return std_device(device)
