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
    return nn.Sequential(*layers)


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


@pytest.mark.parametrize("mode", [1, 3, 0, 2])
def test_fused_linear_is_the_composed_form_bit_for_bit(nt, mode):
    """nn.Linear's one-call path (bias added in the GEMM epilogue in mode 1, by an in-place add in the
    other modes) against matmul followed by a broadcast add: forward and all three gradients."""
    import nanotorch_b200.nn as nn

    rng = np.random.default_rng(77)
    nt._C.set_matmul_mode(mode)
    try:
        for m, k, n in [(64, 48, 10), (257, 100, 130), (512, 256, 384), (1000, 64, 4096)]:
            layer = nn.Linear(k, n)
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
