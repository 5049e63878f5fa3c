"""Modules and the SGD optimizer: the callers of the op kernels in the MLP configurations.

Mirror of the reference's ``nanotorch.nn`` (src/nanotorch/nn/module.py:14-125,
src/nanotorch/nn/optimizers.py:9-51) with the same class and method names.  ``Linear`` draws its
weights from the same seeded host stream with the same expression, so ``manual_seed(0)`` gives the
reference's parameters value for value.
"""

from __future__ import annotations

import math
from typing import Any, Sequence

from . import _C, compute_on_device, rand, zeros
from .autograd import LinearOp, ReluOp, TanhOp, no_grad
from .tensor import Tensor
from ._C import Device, Dtype


class Module:
    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self.forward(*args, **kwargs)

    def parameters(self) -> Sequence[Tensor]:
        return []

    def to(self, device: Device | str) -> "Module":
        return self

    def forward(self, *args: Any, **kwargs: Any) -> Any:
        raise NotImplementedError


def _kaiming_W(fan_in: int, fan_out: int, device) -> Tensor:
    """2 * U[0,1) * z - z with z = sqrt(6 / fan_in): three rounded fp32 kernels, as in the reference
    (src/nanotorch/nn/module.py:118-125)."""
    if fan_in <= 0 or fan_out <= 0:
        raise ValueError(f"Cannot initialize Linear with {fan_in=}, {fan_out=} (non-positive).")
    z = math.sqrt(6 / fan_in)
    return compute_on_device(rand(fan_in, fan_out, device=device), lambda u: 2 * u * z - z)


class Linear(Module):
    """x @ W + b with W of shape (fan_in, fan_out).

    Built on the Cpu and moved with ``.to(device)``, as in the reference (src/nanotorch/nn/module.py:45-63);
    ``device`` (an addition) builds the parameters in place on that device instead."""

    def __init__(self, fan_in: int, fan_out: int, bias: bool = True, device: Device | str = Device.Cpu) -> None:
        with no_grad():
            self._W = _kaiming_W(fan_in, fan_out, device)
        self._W.enable_grad()
        self._b = zeros(fan_out, requires_grad=True, device=device) if bias else None

    def parameters(self) -> Sequence[Tensor]:
        return [self._W] if self._b is None else [self._W, self._b]

    def to(self, device: Device | str) -> "Linear":
        self._W = self._W.to(device)
        if self._b is not None:
            self._b = self._b.to(device)
        return self

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim != 2:
            raise NotImplementedError(f"Can only forward a 2D tensor for now, got {x.ndim}")
        if x.shape[1] != self._W.shape[0]:
            raise ValueError(f"Cannot align axes of size {x.shape[1]} and {self._W.shape[0]}.")
        if self._b is not None and LinearOp.applicable(x, self._W, self._b):
            return LinearOp.apply(x, self._W, self._b)  # same bits as the two steps below, one launch fewer
        z = x @ self._W
        if self._b is not None:
            z = z + self._b
        return z


class ReLU(Module):
    def forward(self, x: Tensor) -> Tensor:
        return ReluOp.apply(x)


class Tanh(Module):
    def forward(self, x: Tensor) -> Tensor:
        return TanhOp.apply(x)


class Sequential(Module):
    def __init__(self, *modules: Module) -> None:
        self._modules = list(modules)

    def parameters(self) -> Sequence[Tensor]:
        return [p for m in self._modules for p in m.parameters()]

    def to(self, device: Device | str) -> "Sequential":
        self._modules = [m.to(device) for m in self._modules]
        return self

    def forward(self, *args: Any, **kwargs: Any) -> Any:
        x = self._modules[0](*args, **kwargs)
        for m in self._modules[1:]:
            x = m(x)
        return x


class Optimizer:
    def __init__(self, parameters: Sequence[Tensor]) -> None:
        self._parameters = parameters

    @property
    def parameters(self) -> Sequence[Tensor]:
        return self._parameters

    def zero_grad(self) -> None:
        for p in self._parameters:
            p.zero_grad()

    def step(self) -> None:
        raise NotImplementedError


class GradientDescent(Optimizer):
    """p <- p - (grad * lr), per parameter.

    Float32 parameters on Cuda take one fused kernel with the two roundings of the reference's
    ``p -= p.grad * lr`` (src/nanotorch/nn/optimizers.py:45-51); anything else runs that expression.
    ``grad_scale`` multiplies the gradient first (1/world_size in data-parallel training).
    """

    def __init__(self, parameters: Sequence[Tensor], lr: float, grad_scale: float = 1.0) -> None:
        super().__init__(parameters)
        self._lr = lr
        self._grad_scale = grad_scale

    def step(self) -> None:
        for p in self.parameters:
            if not p.requires_grad:
                continue
            if p.grad is None:
                raise RuntimeError("Gradients not set, did you call backward?")
            g = p.grad
            if (p.dtype == Dtype.Float32 and g.dtype == Dtype.Float32 and p.device == Device.Cuda
                    and g.shape == p.shape):
                _C.sgd_update(p._C_view, g._C_view, self._lr, self._grad_scale)
            else:
                with no_grad():
                    if self._grad_scale != 1.0:
                        g = g * self._grad_scale
                    p -= g * self._lr
