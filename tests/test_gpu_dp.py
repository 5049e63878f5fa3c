"""Data-parallel training on two GPUs against the same training on one (skipped with < 2 GPUs).

Each rank is a child process driving one GPU; gradients cross NVLink through NCCL only.  The ranks
leave only after their last step, with no kernel or collective in flight.  NVLS is switched off for
the test (a rank that died while bound to an NVLink multicast object has raised faults on its peers
on shared machines)."""

import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent(r"""
    import os, sys
    import numpy as np
    sys.path.insert(0, os.environ["NT_REPO"])
    import nanotorch_b200 as nt
    import nanotorch_b200.nn as nn
    from nanotorch_b200 import _C
    from nanotorch_b200.dp import Communicator, DataParallelSGD, shard_bounds

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    _C.set_device(int(os.environ["LOCAL_RANK"]))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world)

    def exchange(uid):
        box = [uid]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    comm = Communicator(rank, world, exchange)
    dims = [96, 128, 128, 64]
    nt.manual_seed(0)
    layers = []
    for i in range(3):
        layers.append(nn.Linear(dims[i], dims[i + 1]))
        if i < 2:
            layers.append(nn.Tanh())
    model = nn.Sequential(*layers).to("cuda")
    B = 512
    X = np.random.default_rng(40).standard_normal((B, dims[0])).astype(np.float32)
    Y = np.random.default_rng(41).standard_normal((B, dims[-1])).astype(np.float32)
    lo, hi = shard_bounds(B, rank, world)
    tX, tY = nt.Tensor.from_numpy(X[lo:hi], "cuda"), nt.Tensor.from_numpy(Y[lo:hi], "cuda")
    opt = DataParallelSGD(model.parameters(), 1e-2, comm)
    losses = []
    for _ in range(6):
        loss = nt.mean((model(tX) - tY) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.numpy()))
    nt.sync()
    if dist is not None:   # global loss = mean of the equal-sized shards' losses
        import torch
        t = torch.tensor(losses, dtype=torch.float64)
        dist.all_reduce(t)
        losses = (t / world).tolist()
    if rank == 0:
        np.savez(os.environ["NT_OUT"], losses=np.array(losses), **{f"p{i}": p.numpy() for i, p in enumerate(model.parameters())})
    if dist is not None:
        dist.barrier()
    comm.close()
    if dist is not None:
        dist.destroy_process_group()
    print(f"rank {rank} ok")
""")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world: int, script: Path, out: Path):
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NT_REPO=str(REPO), NT_OUT=str(out), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=600)[0])
    except subprocess.TimeoutExpired:
        for p in procs:  # leave no rank behind on the shared GPUs
            p.kill()
            p.wait()
        raise
    for rank, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} of {world} failed:\n{o[-3000:]}"
    return np.load(out)


def test_two_ranks_match_one(nt, tmp_path):
    if nt._C.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    one = _run(1, script, tmp_path / "one.npz")
    two = _run(2, script, tmp_path / "two.npz")
    # same model, same global batch: only the summation order of the gradients differs
    assert np.abs(one["losses"] - two["losses"]).max() <= 1e-5 * np.abs(one["losses"]).max()
    assert one["losses"][-1] < one["losses"][0]
    for k in one.files:
        if k.startswith("p"):
            assert np.abs(one[k] - two[k]).max() <= 1e-5 * (np.abs(one[k]).max() + 1e-3), k
