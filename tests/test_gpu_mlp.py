"""GPU parity of whole training steps against the reference's own runs (golden fixtures)."""

import numpy as np
import pytest

from tests.util import assert_bit_exact, assert_scaled

pytestmark = pytest.mark.gpu


def build(nt, dims, act):
    import nanotorch_b200.nn as nn

    nt.manual_seed(0)
    layers = []
    for i in range(len(dims) - 1):
        layers.append(nn.Linear(dims[i], dims[i + 1]))
        if i < len(dims) - 2:
            layers.append(act())
    return nn.Sequential(*layers).to("cuda")  # built on the Cpu and moved, as the reference's scripts do


@pytest.mark.parametrize("mode", [2, 0, 1])
def test_configuration_1(nt, golden, mode):
    """784 -> 256 -> 10, ReLU, MSE, batch 256, seed-0 Kaiming init, SGD lr 0.01, 100 steps."""
    import nanotorch_b200.nn as nn

    nt._C.set_matmul_mode(mode)
    try:
        model = build(nt, [784, 256, 10], nn.ReLU)
        assert_bit_exact(model.parameters()[0].numpy()[0, :8], golden["mlp1/W1_head"], "seed-0 init")
        X = nt.Tensor.from_numpy(np.random.default_rng(1).standard_normal((256, 784)).astype(np.float32), "cuda")
        Y = nt.Tensor.from_numpy(np.random.default_rng(2).standard_normal((256, 10)).astype(np.float32), "cuda")
        opt = nn.GradientDescent(model.parameters(), lr=0.01)
        losses = []
        for _ in range(100):
            loss = nt.mean((model(X) - Y) ** 2)
            opt.zero_grad()
            loss.backward()
            opt.step()
            losses.append(loss)
        got = np.array([l.numpy() for l in losses], np.float32).reshape(-1)
    finally:
        nt._C.set_matmul_mode(1)
    want = golden["mlp1/losses"]
    rel = np.abs(got - want) / want
    print(f"mode {mode}: loss[0] {got[0]:.7f} (ref {want[0]:.7f}), loss[99] {got[99]:.7f} (ref {want[99]:.7f}), "
          f"max rel diff {rel.max():.2e}")
    assert rel.max() < 1e-4
    assert_scaled(model.parameters()[2].numpy(), golden["mlp1/W2_final"], np.abs(golden["mlp1/W2_final"]).max(), 1e-4, "W2")
    assert_scaled(model.parameters()[1].numpy(), golden["mlp1/b1_final"], np.abs(golden["mlp1/b1_final"]).max() + 1e-3, 1e-3, "b1")


@pytest.mark.parametrize("mode", [2, 1])
def test_tanh_network_gradients(nt, golden, mode):
    """Linear/Tanh x3 + Linear (the shape of the data-parallel configuration, small): first-step
    gradients of every parameter and the 5-step loss curve."""
    import nanotorch_b200.nn as nn

    nt._C.set_matmul_mode(mode)
    try:
        model = build(nt, [24, 32, 32, 32, 16], nn.Tanh)
        X = nt.Tensor.from_numpy(golden["mlp5s/X"], "cuda")
        Y = nt.Tensor.from_numpy(golden["mlp5s/Y"], "cuda")
        opt = nn.GradientDescent(model.parameters(), lr=1e-3)
        losses = []
        for step in range(5):
            loss = nt.mean((model(X) - Y) ** 2)
            opt.zero_grad()
            loss.backward()
            if step == 0:
                for i, p in enumerate(model.parameters()):
                    want = golden[f"mlp5s/grad0/{i}"]
                    assert_scaled(p.grad.numpy(), want, np.abs(want).max(), 1e-4, f"grad of parameter {i}")
            opt.step()
            losses.append(float(loss.numpy()))
    finally:
        nt._C.set_matmul_mode(1)
    want = golden["mlp5s/losses"]
    assert np.abs(np.array(losses) - want).max() / want.max() < 1e-5
    for i, p in enumerate(model.parameters()):
        w = golden[f"mlp5s/final/{i}"]
        assert_scaled(p.numpy(), w, np.abs(w).max() + 1e-6, 1e-4, f"parameter {i} after 5 steps")


def test_captured_step_replays_bit_exact(nt):
    """One training step captured into a CUDA graph and replayed equals the same steps issued eagerly,
    bit for bit, and eager work in between is never given memory the graph writes."""
    import nanotorch_b200.nn as nn

    X = nt.Tensor.from_numpy(np.random.default_rng(1).standard_normal((256, 96)).astype(np.float32), "cuda")
    Y = nt.Tensor.from_numpy(np.random.default_rng(2).standard_normal((256, 32)).astype(np.float32), "cuda")

    def run(graph_mode: bool):
        model = build(nt, [96, 160, 160, 32], nn.Tanh)
        opt = nn.GradientDescent(model.parameters(), lr=1e-2)

        def step():
            loss = nt.mean((model(X) - Y) ** 2)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss

        losses = [float(step().numpy()) for _ in range(2)]  # warm-up, eager in both runs
        if graph_mode:
            g = nt._C.Graph()
            with g.capture():
                loss = step()
            # capture only records: the parameters have not moved yet
            for _ in range(4):
                g.replay()
                noise = (X * 3.0).sum()            # eager work between replays, allocating and freeing
                losses.append(float(loss.numpy()))
                del noise
            g.close()
        else:
            losses += [float(step().numpy()) for _ in range(4)]
        return np.array(losses), [p.numpy() for p in model.parameters()]

    eager_losses, eager_params = run(False)
    graph_losses, graph_params = run(True)
    assert np.array_equal(eager_losses, graph_losses), (eager_losses, graph_losses)
    for a, b in zip(eager_params, graph_params):
        assert_bit_exact(a, b, "parameters after replayed steps")


def test_replayed_step_reads_the_batch_its_buffers_hold_now(nt):
    """A captured step is fed by writing the next batch into the same input buffers before each replay.
    The split planes of an input that an eager warm-up step left behind must not be what the graph reads:
    losses and parameters equal the eager run over the same sequence of batches, bit for bit."""
    import nanotorch_b200.nn as nn

    rng = np.random.default_rng(7)
    xs = [rng.standard_normal((512, 640)).astype(np.float32) for _ in range(5)]
    ys = [rng.standard_normal((512, 64)).astype(np.float32) for _ in range(5)]

    def run(graph_mode: bool):
        X = nt.Tensor.from_numpy(xs[0], "cuda")
        Y = nt.Tensor.from_numpy(ys[0], "cuda")
        model = build(nt, [640, 768, 64], nn.Tanh)
        opt = nn.GradientDescent(model.parameters(), lr=1e-2)

        def feed(i):
            X.storage.upload(xs[i].ctypes.data, xs[i].nbytes)
            Y.storage.upload(ys[i].ctypes.data, ys[i].nbytes)

        def step():
            loss = nt.mean((model(X) - Y) ** 2)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss

        losses = [float(step().numpy())]                  # eager warm-up on batch 0
        if graph_mode:
            g = nt._C.Graph()
            with g.capture():
                loss = step()
            for i in range(1, 5):
                feed(i)
                g.replay()
                losses.append(float(loss.numpy()))
            g.close()
        else:
            for i in range(1, 5):
                feed(i)
                losses.append(float(step().numpy()))
        return np.array(losses), [p.numpy() for p in model.parameters()]

    eager_losses, eager_params = run(False)
    graph_losses, graph_params = run(True)
    assert len(set(eager_losses.tolist())) == 5
    assert np.array_equal(eager_losses, graph_losses), (eager_losses, graph_losses)
    for a, b in zip(eager_params, graph_params):
        assert_bit_exact(a, b, "parameters after replays over fresh batches")


@pytest.mark.parametrize("graph_mode", [False, True])
def test_side_stream_update_equals_plain_sgd(nt, graph_mode):
    """DataParallelSGD with one rank: no collective, but every bucket's update runs on the communication
    stream the moment backward has finished that bucket's gradients.  Same bits as GradientDescent after
    six steps, eagerly and as a replayed CUDA graph (the cross-stream edges are part of the capture)."""
    import nanotorch_b200.nn as nn
    from nanotorch_b200.dp import Communicator, DataParallelSGD

    X = nt.Tensor.from_numpy(np.random.default_rng(1).standard_normal((512, 640)).astype(np.float32), "cuda")
    Y = nt.Tensor.from_numpy(np.random.default_rng(2).standard_normal((512, 64)).astype(np.float32), "cuda")

    def run(side: bool):
        model = build(nt, [640, 768, 768, 64], nn.Tanh)
        if side:
            opt = DataParallelSGD(model.parameters(), 1e-2, Communicator(0, 1, None))
            assert [len(b) for b in opt._buckets] == [2, 2, 2]
        else:
            opt = nn.GradientDescent(model.parameters(), lr=1e-2)

        def step():
            loss = nt.mean((model(X) - Y) ** 2)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss

        losses = [float(step().numpy()) for _ in range(2)]
        if side and graph_mode:
            g = nt._C.Graph()
            with g.capture():
                loss = step()
            for _ in range(4):
                g.replay()
                losses.append(float(loss.numpy()))
            g.close()
        else:
            losses += [float(step().numpy()) for _ in range(4)]
        if side:
            opt.detach()
        return np.array(losses), [p.numpy() for p in model.parameters()]

    plain_losses, plain_params = run(False)
    side_losses, side_params = run(True)
    assert np.array_equal(plain_losses, side_losses), (plain_losses, side_losses)
    for a, b in zip(plain_params, side_params):
        assert_bit_exact(a, b, "parameters after six steps")


def test_training_script_flow(nt):
    """The steps of the reference's training script (scripts/train_mlp_basic.py:30-58) as it writes them:
    data made on the Cpu and moved, a matrix @ 1-D product for the targets, modules built on the Cpu and
    moved with .to(device), batches taken by slicing, squeeze() on the prediction, the loss read with
    .cpu().item().  The loss must fall."""
    import nanotorch_b200.nn as nn

    nt.manual_seed(3)
    device = "cuda"
    n, f, h, bs = 4096, 64, 64, 512
    X = nt.rand(n, f).to(device)
    y = (X @ nt.randint(-10, 10, (f,)).to(device) + 3.14).to(device)
    model = nn.Sequential(nn.Linear(f, h), nn.ReLU(), nn.Linear(h, h), nn.Tanh(), nn.Linear(h, 1)).to(device)
    optimizer = nn.GradientDescent(model.parameters(), lr=1e-4)
    first = last = None
    for _ in range(3):
        for i in range(0, n, bs):
            xb, yb_true = X[i:i + bs], y[i:i + bs]
            yb_pred = model(xb)
            loss = nt.mean((yb_pred.squeeze() - yb_true) ** 2)
            optimizer.zero_grad()
            loss.backward()
            optimizer.step()
            last = loss.cpu().item()
            first = last if first is None else first
    assert np.isfinite(last) and last < first
    assert isinstance(yb_true[0].cpu().item(), float) and isinstance(yb_pred[0].cpu().item(), float)


@pytest.mark.parametrize("mode", [1, 3, 0, 2])
def test_fused_linear_is_the_composed_form_bit_for_bit(nt, mode):
    """nn.Linear's one-call path (bias added in the GEMM epilogue in mode 1, by an in-place add in the
    other modes) against matmul followed by a broadcast add: forward and all three gradients."""
    import nanotorch_b200.nn as nn

    rng = np.random.default_rng(77)
    nt._C.set_matmul_mode(mode)
    try:
        for m, k, n in [(64, 48, 10), (257, 100, 130), (512, 256, 384), (1000, 64, 4096)]:
            layer = nn.Linear(k, n, device="cuda")
            W, b = layer.parameters()
            with nt.no_grad():
                b += nt.Tensor.from_numpy(rng.standard_normal(n).astype(np.float32), "cuda")  # a non-zero bias
            x_np = rng.standard_normal((m, k)).astype(np.float32)
            g_np = rng.standard_normal((m, n)).astype(np.float32)
            grads = []
            outs = []
            for fused in (True, False):
                x = nt.Tensor.from_numpy(x_np, "cuda", requires_grad=True)
                for p in (W, b):
                    p.zero_grad()
                z = layer(x) if fused else (x @ W) + b
                assert (z.grad_fn.__class__.__name__ == "LinearOp") == fused
                (z * nt.Tensor.from_numpy(g_np, "cuda")).sum().backward()
                outs.append(z.numpy())
                grads.append((x.grad.numpy(), W.grad.numpy(), b.grad.numpy()))
            assert_bit_exact(outs[0], outs[1], f"forward {m}x{k}x{n} mode {mode}")
            for got, want, what in zip(grads[0], grads[1], ("dX", "dW", "db")):
                assert_bit_exact(got, want, f"{what} {m}x{k}x{n} mode {mode}")
        # a strided bias view and the raw entry point's checks
        W = nt.Tensor.from_numpy(rng.standard_normal((32, 20)).astype(np.float32), "cuda")
        x = nt.Tensor.from_numpy(rng.standard_normal((16, 32)).astype(np.float32), "cuda")
        wide = nt.Tensor.from_numpy(rng.standard_normal((40,)).astype(np.float32), "cuda")
        got = nt.Tensor._new_contiguous(nt._C.linear(x._C_view, W._C_view, wide[::2]._C_view), (16, 20))
        assert_bit_exact(got.numpy(), ((x @ W) + wide[::2]).numpy(), "strided bias")
        with pytest.raises(ValueError):
            nt._C.linear(x._C_view, W._C_view, wide._C_view)
    finally:
        nt._C.set_matmul_mode(1)


@pytest.mark.parametrize("graph_mode", [False, True])
def test_overlapped_gradient_products_leave_the_step_unchanged(nt, graph_mode):
    """Linear.backward launches its two products as an overlapping pair: six training steps, eagerly and as a
    replayed graph, give the bits of the same steps with the overlap switched off."""
    import nanotorch_b200.nn as nn

    X = nt.Tensor.from_numpy(np.random.default_rng(1).standard_normal((2048, 1024)).astype(np.float32), "cuda")
    Y = nt.Tensor.from_numpy(np.random.default_rng(2).standard_normal((2048, 256)).astype(np.float32), "cuda")

    def run(overlap: bool):
        nt._C.set_matmul_pair_overlap(overlap)
        try:
            model = build(nt, [1024, 1536, 1536, 256], nn.Tanh)
            opt = nn.GradientDescent(model.parameters(), lr=1e-2)

            def step():
                loss = nt.mean((model(X) - Y) ** 2)
                opt.zero_grad()
                loss.backward()
                opt.step()
                return loss

            losses = [float(step().numpy()) for _ in range(2)]
            if graph_mode:
                g = nt._C.Graph()
                with g.capture():
                    loss = step()
                for _ in range(4):
                    g.replay()
                    losses.append(float(loss.numpy()))
                g.close()
            else:
                losses += [float(step().numpy()) for _ in range(4)]
            return np.array(losses), [p.numpy() for p in model.parameters()]
        finally:
            nt._C.set_matmul_pair_overlap(False)

    plain_losses, plain_params = run(False)
    pair_losses, pair_params = run(True)
    assert np.array_equal(plain_losses, pair_losses), (plain_losses, pair_losses)
    for a, b in zip(plain_params, pair_params):
        assert_bit_exact(a, b, "parameters after six steps")
