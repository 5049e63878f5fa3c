"""Host logic of the data-parallel path on CPU ranks over gloo: shard bounds, the exchange of the
communicator id, bucketed hook-driven exchange + update ordering, the once-per-pass hook contract
(shared parameters, a second backward pass), the averaging identity the step relies on (sum of
local-mean gradients / world == gradient of the global-batch mean), and failure detection on the host:
a rank that leaves between steps is found by the survivor within the stated limit instead of a hang,
and a rendezvous or exchange that overruns its limit becomes an error."""

import os
import socket
import subprocess
import sys
import textwrap
import time
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent

MOCKS = textwrap.dedent(r"""
    import os, sys
    import numpy as np
    sys.path.insert(0, os.environ["NT_REPO"])
    import nanotorch_b200 as nt
    from nanotorch_b200 import dp, _C
    from nanotorch_b200.autograd import leaf_grad_hooks

    calls = []
    _C.comm_unique_id = lambda: bytes(range(128))
    _C.comm_init = lambda r, w, uid: calls.append(("init", r, w, uid))
    _C.comm_init_timeout = lambda r, w, uid, ms: calls.append(("init_timeout", r, w, uid, ms))
    _C.comm_group_begin = lambda: calls.append(("group_begin",))
    _C.comm_group_end = lambda: calls.append(("group_end",))
    _C.comm_allreduce_sum = lambda storage: calls.append(("allreduce", storage.size))
    _C.comm_sgd_update = lambda p, g, lr, scale=1.0: calls.append(("sgd", tuple(p.shape), lr, scale))
    _C.comm_wait = lambda: calls.append(("wait",))
    _C.comm_destroy = lambda: calls.append(("destroy",))
    _C.comm_abort = lambda: calls.append(("abort",))
""")

WORKER = MOCKS + textwrap.dedent(r"""
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world)

    def exchange(uid):
        box = [uid]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    # ---- the communicator: id made on rank 0 only, broadcast over the host channel, same bytes everywhere
    comm = dp.Communicator(rank, world, exchange)
    assert calls == [("init", rank, world, bytes(range(128)))], calls
    del calls[:]

    # ---- buckets: a weight and the bias declared after it share one; exchange + update of a bucket are
    # issued the moment its last gradient is final, in the order backward reaches the layers
    big = 600 * 600  # 1.44 MB of fp32: worth a launch of its own
    params = [nt.zeros(600, 600, requires_grad=True), nt.zeros(600, requires_grad=True),
              nt.zeros(600, 600, requires_grad=True), nt.zeros(600, requires_grad=True)]
    opt = dp.DataParallelSGD(params, 0.1, comm)
    assert [len(b) for b in opt._buckets] == [2, 2]
    assert set(leaf_grad_hooks) == {id(p) for p in params}
    opt._update = lambda p, on_side_stream: calls.append(("update", p.numel, on_side_stream))
    for p in (params[2], params[3], params[0], params[1]):   # backward reaches the last layer first
        p._grad = nt.zeros(*p.shape)
        leaf_grad_hooks[id(p)](p)
    one = [("group_begin",), ("allreduce", big), ("allreduce", 600), ("group_end",), ("update", big, True), ("update", 600, True)]
    assert calls == one + one, calls
    # a second backward pass before step() would accumulate into gradients that are already on the wire
    try:
        leaf_grad_hooks[id(params[0])](params[0])
        raise SystemExit("second pass was not rejected")
    except RuntimeError as e:
        assert "second backward pass" in str(e)
    del calls[:]
    opt.step()
    assert calls == [("wait",)] and opt._grad_scale == 1.0 / world
    opt.detach()
    assert not leaf_grad_hooks

    # ---- sharding + averaging identity on a linear least-squares model
    B, D = 22, 5
    rng = np.random.default_rng(0)
    X, Y, W = rng.standard_normal((B, D)), rng.standard_normal((B, 1)), rng.standard_normal((D, 1))
    lo, hi = dp.shard_bounds(B, rank, world)
    bounds = [None] * world
    dist.all_gather_object(bounds, (lo, hi))
    assert bounds[0][0] == 0 and bounds[-1][1] == B and all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
    Xl, Yl = X[lo:hi], Y[lo:hi]
    g_local = torch.from_numpy(2 * Xl.T @ (Xl @ W - Yl) / (hi - lo))   # gradient of the LOCAL mean
    # ranks hold equal shards here (22 = 11 + 11); with unequal shards the weights are the shard sizes
    assert hi - lo == B // world
    dist.all_reduce(g_local)
    g_avg = g_local.numpy() / world
    g_global = 2 * X.T @ (X @ W - Y) / B
    assert np.allclose(g_avg, g_global, rtol=1e-12), (g_avg, g_global)

    # ---- max over ranks of a timing, as the benchmark takes it
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == 10.0 + world - 1
    comm.close()
    assert calls[-1] == ("destroy",)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")
""")

# One rank leaves between steps (host-side failure, nothing in flight); the survivor must learn of it
# on the host within the monitor's limit, abort its communicator and return an error -- not hang.
LEAVER = MOCKS + textwrap.dedent(r"""
    import time
    from datetime import timedelta
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, is_master=(rank == 0),
                          timeout=timedelta(seconds=30))
    comm = dp.Communicator(rank, world, lambda uid: uid or bytes(range(128)), timeout_s=20.0)
    assert calls[0][0] == "init_timeout" and calls[0][-1] == 20000
    monitor = dp.PeerMonitor(store, rank, world, timeout_s=2.0)
    steps = 0
    try:
        for step in range(5):
            monitor.await_peers(steps)          # everyone finished the previous step
            if rank == 1 and step == 2:
                print("rank 1 leaves", flush=True)
                sys.exit(0)                     # between steps: no kernel, no collective in flight
            steps = monitor.report()
        raise SystemExit("the survivor never noticed")
    except dp.PeerLost as e:
        comm.abort()
        assert calls[-1] == ("abort",)
        print(f"rank {rank} detected: {e}", flush=True)
""")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(script: Path, world: int, port: int):
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NT_REPO=str(REPO))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    return procs


def _collect(procs, timeout):
    outputs = []
    try:
        for p in procs:
            outputs.append(p.communicate(timeout=timeout)[0])
    except subprocess.TimeoutExpired:
        for p in procs:
            p.kill()
            p.wait()
        raise
    return outputs


def test_two_rank_host_logic(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = _spawn(script, 2, _free_port())
    outputs = _collect(procs, 180)
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out


def test_rank_that_leaves_between_steps_is_detected_on_the_host(tmp_path):
    script = tmp_path / "leaver.py"
    script.write_text(LEAVER)
    t0 = time.monotonic()
    procs = _spawn(script, 2, _free_port())
    outputs = _collect(procs, 120)
    assert procs[1].returncode == 0 and "rank 1 leaves" in outputs[1], outputs[1]
    assert procs[0].returncode == 0, outputs[0]
    assert "rank 0 detected: rank 1 reported 2 finished steps, 3 expected" in outputs[0], outputs[0]
    assert time.monotonic() - t0 < 60  # the monitor's limit is 2 s; nothing waited on a collective


def test_hook_fires_once_per_pass_for_a_shared_parameter():
    """The backward engine calls a leaf's hook once, after the last contribution (a parameter used
    twice in the graph gets one call, with the summed gradient already in place)."""
    import nanotorch_b200 as nt
    from nanotorch_b200.autograd import Function, leaf_grad_hooks

    class Twice(Function):   # y = 2 * x without a kernel: backward hands the upstream gradient on
        def forward(self, x):
            return nt.Tensor._new_view(x.storage, x.shape, x._strides, x._offset)

        def backward(self, g):
            return (g,)

    w = nt.Tensor([1.0, 2.0], requires_grad=True)
    a, b = Twice.apply(w), Twice.apply(w)
    seen = []

    class Join(Function):
        def forward(self, x, y):
            return nt.Tensor._new_view(x.storage, x.shape, x._strides, x._offset)

        def backward(self, g):
            return g, g

    out = Join.apply(a, b)
    leaf_grad_hooks[id(w)] = lambda p: seen.append(p.grad)
    try:
        import nanotorch_b200.tensor as T

        class FakeGrad:  # stands in for a device gradient: counts the accumulations
            def __init__(self, n=1):
                self.n = n

            def __add__(self, other):
                return FakeGrad(self.n + other.n)

        out._grad = FakeGrad()
        from nanotorch_b200.autograd import run_backward

        run_backward(out)
    finally:
        leaf_grad_hooks.pop(id(w), None)
    assert len(seen) == 1 and seen[0].n == 2


def test_exchange_time_limits_are_plumbed(monkeypatch):
    """Communicator(timeout_s=...) bounds the rendezvous, sync(timeout) the outstanding collectives,
    abort() is reachable: the native calls are replaced by recorders, the units checked."""
    from nanotorch_b200 import _C, dp

    calls = []
    monkeypatch.setattr(_C, "comm_unique_id", lambda: bytes(128))
    monkeypatch.setattr(_C, "comm_init_timeout", lambda r, w, uid, ms: calls.append(("init", r, w, ms)))
    monkeypatch.setattr(_C, "comm_sync", lambda ms: calls.append(("sync", ms)))
    monkeypatch.setattr(_C, "comm_abort", lambda: calls.append(("abort",)))
    comm = dp.Communicator(0, 2, lambda uid: uid, timeout_s=1.5)
    comm.sync(0.25)
    comm.abort()
    assert calls == [("init", 0, 2, 1500), ("sync", 250), ("abort",)]

    def overrun(ms):
        raise RuntimeError(f"nt_comm_sync: collectives still outstanding after {ms} ms; the communicator was aborted.")

    monkeypatch.setattr(_C, "comm_sync", overrun)
    with pytest.raises(RuntimeError, match="still outstanding after 100 ms"):
        comm.sync(0.1)
