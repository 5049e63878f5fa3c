"""Host logic of the data-parallel path on two CPU ranks over gloo: shard bounds, the exchange of
the communicator id, hook-driven all-reduce ordering, and the averaging identity the step relies on
(sum of local-mean gradients / world == gradient of the global-batch mean)."""

import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent(r"""
    import os, sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.environ["NT_REPO"])
    import nanotorch_b200 as nt
    from nanotorch_b200 import dp, _C
    from nanotorch_b200.autograd import leaf_grad_hooks

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world)

    # ---- the communicator: id made on rank 0 only, broadcast over the host channel, same bytes everywhere
    calls = []
    _C.comm_unique_id = lambda: bytes(range(128))
    _C.comm_init = lambda r, w, uid: calls.append(("init", r, w, uid))
    _C.comm_allreduce_sum = lambda storage: calls.append(("allreduce", storage.size))
    _C.comm_wait = lambda: calls.append(("wait",))
    _C.comm_destroy = lambda: calls.append(("destroy",))

    def exchange(uid):
        box = [uid]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    comm = dp.Communicator(rank, world, exchange)
    assert calls == [("init", rank, world, bytes(range(128)))], calls

    # ---- hooks: one all-reduce per parameter, in the order backward produces the gradients
    params = [nt.Tensor([[1.0, 2.0], [3.0, 4.0]], requires_grad=True), nt.Tensor([0.5, 0.25], requires_grad=True)]
    sgd_calls = []
    _C.sgd_update = lambda p, g, lr, scale=1.0: sgd_calls.append((tuple(p.shape), lr, scale))
    opt = dp.DataParallelSGD(params, 0.1, comm)
    assert set(leaf_grad_hooks) == {id(p) for p in params}
    for p in reversed(params):          # backward reaches the last layer's parameters first
        p._grad = nt.Tensor([[0.0] * 2] * 2) if p.ndim == 2 else nt.Tensor([0.0] * 2)
        leaf_grad_hooks[id(p)](p)
    assert calls[1:] == [("allreduce", 2), ("allreduce", 4)], calls
    # the update waits for the collectives and folds 1/world into the step (a CPU parameter takes
    # the generic path; only the ordering and the scale are checked here)
    assert opt._grad_scale == 1.0 / world
    opt._comm.wait()
    assert calls[-1] == ("wait",)
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


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_host_logic(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NT_REPO=str(REPO))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outputs = [p.communicate(timeout=180)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out
