"""Device handling.

The first three functions are the reference's ``nanotorch.cuda`` module (src/nanotorch/cuda.py), which
its scripts call as ``nt.cuda.is_available()`` / ``nt.cuda.sync()``.  The rest exposes what this library
adds around the device: one process drives one GPU, chosen before the first allocation; every kernel runs
on one library-owned stream; device memory comes from a caching arena.
"""

from typing import Literal

from . import _C
from .tensor import std_device

Device = _C.Device
DeviceLiteral = Literal["cpu", "cuda"]

is_available = _C.is_cuda_available   # a CUDA device is present and usable
sync = _C.cuda_sync                   # wait for everything enqueued on the library's stream
get_std_device = std_device           # "cpu" / "cuda" / Device -> Device, ValueError otherwise


def device_count() -> int:
    """Number of visible CUDA devices."""
    return _C.device_count()


def set_device(ordinal: int) -> None:
    """Bind this process to one GPU; call before the first device allocation (one process per GPU)."""
    _C.set_device(ordinal)


def stream() -> int:
    """The ``cudaStream_t`` (as an integer) that every kernel of the library is launched on."""
    return _C.stream_handle()


def launches() -> int:
    """Kernels launched by the library since it was loaded."""
    return _C.launch_count()


def memory_stats() -> dict:
    """Bytes reserved from the driver / in use / number of ``cudaMalloc`` calls of the caching arena."""
    return _C.allocator_stats()


def empty_cache() -> None:
    """Return the arena's cached blocks to the driver."""
    _C.allocator_trim()
