"""Data-parallel training over one process per GPU.

The reference is single-device; this is the sharded form of its training step: every rank holds the
same parameters (same seed, same updates), takes a contiguous row block of the global batch, and the
gradient of the global-batch mean is the average of the local gradients.  Each parameter's gradient
is all-reduced (NCCL sum over NVLink) on the communication stream as soon as backward has written
it, while the remaining layers' backward kernels keep running; the 1/world factor is folded into the
SGD kernel.
"""

from __future__ import annotations

from typing import Sequence

from . import _C
from .autograd import leaf_grad_hooks
from .nn import GradientDescent
from .tensor import Tensor


def shard_bounds(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [lo, hi) of `rank`: equal contiguous blocks, remainder spread over the first ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class Communicator:
    """Thin owner of the library's NCCL communicator; `exchange_id` moves the 128-byte id from rank 0
    to the others (any host-side channel: a torch.distributed gloo broadcast, a file, an env var)."""

    def __init__(self, rank: int, world: int, exchange_id):
        self.rank, self.world = rank, world
        if world > 1:
            uid = _C.comm_unique_id() if rank == 0 else None
            uid = exchange_id(uid)
            _C.comm_init(rank, world, uid)

    def allreduce_sum(self, t: Tensor) -> None:
        if self.world > 1:
            if not t._is_contiguous(full_span=True):
                raise RuntimeError("allreduce_sum: gradient must own a dense storage")
            _C.comm_allreduce_sum(t.storage)

    def wait(self) -> None:
        if self.world > 1:
            _C.comm_wait()

    def close(self) -> None:
        if self.world > 1:
            _C.comm_destroy()


class DataParallelSGD(GradientDescent):
    """SGD whose step averages gradients over ranks.

    Registers one hook per parameter: when backward writes that parameter's gradient the all-reduce
    is enqueued immediately (overlapping the rest of backward).  `step` waits for the collectives,
    then applies p <- p - ((g_sum * 1/world) * lr).
    """

    def __init__(self, parameters: Sequence[Tensor], lr: float, comm: Communicator):
        super().__init__(parameters, lr, grad_scale=1.0 / comm.world)
        self._comm = comm
        if comm.world > 1:
            for p in parameters:
                leaf_grad_hooks[id(p)] = self._on_grad

    def _on_grad(self, p: Tensor) -> None:
        g = p.grad
        if not g._is_contiguous(full_span=True):
            g = g._to_contiguous(force=True)
            p._grad = g
        self._comm.allreduce_sum(g)

    def step(self) -> None:
        self._comm.wait()
        super().step()

    def detach(self) -> None:
        for p in self._parameters:
            leaf_grad_hooks.pop(id(p), None)
