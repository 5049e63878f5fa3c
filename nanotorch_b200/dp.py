"""Data-parallel training over one process per GPU.

The reference is single-device; this is the sharded form of its training step: every rank holds the
same parameters (same seed, same updates), takes a contiguous row block of the global batch, and the
gradient of the global-batch mean is the average of the local gradients.

Parameters are grouped into buckets in declaration order (a Linear's weight and bias share one).  The
moment backward has finished the last gradient of a bucket, the bucket's all-reduces (NCCL sum over
NVLink, issued as one NCCL group, i.e. one launch) go to the communication stream, followed -- on a third,
lowest-priority stream, behind the exchange -- by the bucket's SGD kernels with the 1/world factor folded
in.  Exchange and update of one layer thus overlap the backward kernels of the layers below it; `step`
only makes the compute stream wait for the other two.  With one rank there is no collective, and the
updates still run on the side stream, behind the kernels that produced their gradients.
"""

from __future__ import annotations

from typing import Sequence

from . import _C
from ._C import Device, Dtype
from .autograd import leaf_grad_hooks, no_grad
from .nn import GradientDescent
from .tensor import Tensor


def shard_bounds(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [lo, hi) of `rank`: equal contiguous blocks, remainder spread over the first ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class PeerLost(RuntimeError):
    """A peer rank stopped reporting: raised on the host, between steps, before anything is launched."""


class PeerMonitor:
    """Host-side failure detection between steps.

    Every rank counts its finished steps in a shared key-value store (anything with the
    ``add(key, amount) -> int`` of torch.distributed's TCPStore / FileStore / HashStore: an atomic
    increment that also reads).  Before launching step `s` a rank calls ``await_peers(s)``: each peer must
    have reported step `s - 1` within `timeout_s`, else PeerLost names the missing rank.  A rank that
    died or left between steps is thus found on the host, with no kernel or collective in flight, and
    the survivors can abort their communicator and stop (or re-form a smaller group) instead of
    entering a collective that can never complete.
    """

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, poll_s: float = 0.02):
        self._store, self.rank, self.world = store, rank, world
        self._timeout, self._poll = timeout_s, poll_s

    @staticmethod
    def _key(rank: int) -> str:
        return f"nt_b200/steps_done/{rank}"

    def report(self) -> int:
        """This rank finished a step; returns how many it has reported."""
        return int(self._store.add(self._key(self.rank), 1))

    def await_peers(self, steps_done: int) -> None:
        import time

        deadline = time.monotonic() + self._timeout
        for peer in range(self.world):
            if peer == self.rank:
                continue
            while True:
                seen = int(self._store.add(self._key(peer), 0))
                if seen >= steps_done:
                    break
                if time.monotonic() > deadline:
                    raise PeerLost(f"rank {peer} reported {seen} finished steps, {steps_done} expected, "
                                   f"after {self._timeout:.1f} s")
                time.sleep(self._poll)


class Communicator:
    """Thin owner of the library's NCCL communicator; `exchange_id` moves the 128-byte id from rank 0
    to the others (any host-side channel: a torch.distributed gloo broadcast, a file, an env var).
    `timeout_s` bounds the rendezvous: a rank that never joins becomes a RuntimeError, not a hang."""

    def __init__(self, rank: int, world: int, exchange_id, timeout_s: float | None = None):
        self.rank, self.world = rank, world
        if world > 1:
            uid = _C.comm_unique_id() if rank == 0 else None
            uid = exchange_id(uid)
            if timeout_s is None:
                _C.comm_init(rank, world, uid)
            else:
                _C.comm_init_timeout(rank, world, uid, int(timeout_s * 1000))

    def allreduce_sum(self, t: Tensor) -> None:
        if self.world > 1:
            if not t._is_contiguous(full_span=True):
                raise RuntimeError("allreduce_sum: gradient must own a dense storage")
            _C.comm_allreduce_sum(t.storage)

    def wait(self) -> None:
        """The compute stream waits (on the device) for everything on the communication stream."""
        _C.comm_wait()

    def sync(self, timeout_s: float) -> None:
        """Host-side wait for the outstanding collectives with a time limit; past it the communicator is
        aborted and a RuntimeError raised (a peer that died mid-step shows up here)."""
        _C.comm_sync(int(timeout_s * 1000))

    def abort(self) -> None:
        if self.world > 1:
            _C.comm_abort()

    def close(self) -> None:
        if self.world > 1:
            _C.comm_destroy()


class DataParallelSGD(GradientDescent):
    """SGD whose step averages gradients over ranks; exchange and update run bucket by bucket on the
    communication stream while backward continues (see the module docstring).

    A bucket is flushed when every parameter in it has received its final gradient of the pass (the
    backward engine calls the hook once per parameter, after the last contribution).  After the hook
    has fired, no kernel that backward still has to enqueue reads that parameter, which is what makes
    updating it early safe.  One backward pass per step: a second pass before `step` would accumulate
    into gradients whose exchange has already been issued, and raises instead.
    """

    def __init__(self, parameters: Sequence[Tensor], lr: float, comm: Communicator, bucket_bytes: int = 1 << 20):
        super().__init__(parameters, lr, grad_scale=1.0 / comm.world)
        self._comm = comm
        self._buckets: list[list[Tensor]] = []
        self._bucket_of: dict[int, int] = {}
        current, size = [], 0
        for p in parameters:
            if not p.requires_grad:
                continue
            if current and size >= bucket_bytes and p.ndim != 1:
                # a new weight starts a new bucket once the current one is worth a launch; a bias stays
                # with the weight declared just before it
                self._buckets.append(current)
                current, size = [], 0
            current.append(p)
            size += p.numel * 4
        if current:
            self._buckets.append(current)
        for i, b in enumerate(self._buckets):
            for p in b:
                self._bucket_of[id(p)] = i
                leaf_grad_hooks[id(p)] = self._on_grad
        self._ready = [0] * len(self._buckets)
        self._flushed = [False] * len(self._buckets)

    def _on_grad(self, p: Tensor) -> None:
        i = self._bucket_of[id(p)]
        if self._flushed[i]:
            raise RuntimeError("DataParallelSGD: a second backward pass reached a parameter whose gradient exchange "
                               "was already issued; call step() (or zero_grad()) between backward passes.")
        self._ready[i] += 1
        if self._ready[i] == len(self._buckets[i]):
            self._flush(i)

    def _flush(self, i: int) -> None:
        bucket = self._buckets[i]
        for p in bucket:
            g = p.grad
            if not g._is_contiguous(full_span=True):
                g = g._to_contiguous(force=True)
                p._grad = g
        _C.comm_group_begin()
        try:
            for p in bucket:
                self._comm.allreduce_sum(p._grad)
        finally:
            _C.comm_group_end()
        for p in bucket:
            self._update(p, on_side_stream=True)
        self._flushed[i] = True

    def _update(self, p: Tensor, on_side_stream: bool) -> None:
        g = p.grad
        if (p.dtype == Dtype.Float32 and g.dtype == Dtype.Float32 and p.device == Device.Cuda and g.shape == p.shape):
            fn = _C.comm_sgd_update if on_side_stream else _C.sgd_update
            fn(p._C_view, g._C_view, self._lr, self._grad_scale)
        else:
            self._comm.wait()
            with no_grad():
                if self._grad_scale != 1.0:
                    g = g * self._grad_scale
                p -= g * self._lr

    def zero_grad(self) -> None:
        super().zero_grad()
        self._ready = [0] * len(self._buckets)
        self._flushed = [False] * len(self._buckets)

    def step(self) -> None:
        for i, bucket in enumerate(self._buckets):
            if self._flushed[i]:
                continue
            if any(p.grad is None for p in bucket):
                raise RuntimeError("Gradients not set, did you call backward?")
            self._flush(i)  # parameters the hooks did not cover (e.g. gradients assigned by hand)
        self._comm.wait()
        self._ready = [0] * len(self._buckets)
        self._flushed = [False] * len(self._buckets)

    def detach(self) -> None:
        for p in self._parameters:
            leaf_grad_hooks.pop(id(p), None)
