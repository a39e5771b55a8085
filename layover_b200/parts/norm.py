"""RMSNorm and LayerNorm, each fused with the residual addition that precedes it."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, register_norm


@dataclass
class DeferredMean:
    """Several sub-layer outputs that join the stream as `factor` times the sum of their norms (each a
    `Deferred`): the outputs of mixers that run side by side on the same input."""
    parts: tuple
    factor: float


@dataclass
class Deferred:
    """A sub-layer's output that has not joined the residual stream yet because it is RMS-normed
    first (a norm AFTER the sub-layer): the next norm of the stream does both in one kernel,
    x += weight * value * rsqrt(mean(value^2) + eps), then its own norm of x."""
    value: torch.Tensor
    weight: torch.Tensor
    eps: float


@register_norm("rmsnorm")
class RMSNorm(Part):
    """y = weight * round(x * rsqrt(mean(x^2) + eps)), statistics in 32-bit (layover/model.py:25-36).

    params: dim, eps, weight (tensor name relative to the prefix).
    `forward(x, delta)` first adds `delta` into `x` (the residual sum, in 32-bit, rounded once)
    so that a block never launches a separate addition.

    Two more forms, both for models that keep the residual stream in 32-bit floats whatever the
    run's type: `delta` may be a `Deferred` (what `defer(value)` of the norm that FOLLOWS a sub-layer
    returns: its output is normed, then added), and `extra` is one more 32-bit tensor to add (the
    embedding output, between the passes of layers that run several times). These take the
    32-bit-stream kernel, which rounds once, at the output; `add(x, delta, extra)` is the same
    without a norm of the sum."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("dim", "eps", "weight")
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.weight_name = prefix + params["weight"]
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.dim,), kind="vector", init="ones")]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def defer(self, value: torch.Tensor) -> Deferred:
        """`value` as something this norm is to be applied to when it is added to the stream."""
        return Deferred(value, self.weight, self.eps)

    def forward(self, x: torch.Tensor, delta, rows: torch.Tensor | None = None,
                extra: torch.Tensor | None = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        wide = x.dtype == torch.float32 and self.runtime.dtype != torch.float32
        if not (wide or isinstance(delta, Deferred) or extra is not None):
            out = torch.empty((n, self.dim), dtype=x.dtype, device=x.device)
            return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        out = torch.empty((n, self.dim), dtype=self.runtime.dtype, device=x.device)
        value, weight, eps = (delta.value, delta.weight, delta.eps) if isinstance(delta, Deferred) else (delta, None, 0.0)
        return ops.residual_rmsnorm(x, value, weight, eps, extra, self.weight, self.eps, out, rows)

    def forward_after(self, x: torch.Tensor, pending, alpha: float = 1.0, lowered: torch.Tensor | None = None) -> torch.Tensor:
        """The norm AFTER the sum, over a 32-bit stream and in place: x <- norm(alpha * x + pending). `pending` is
        a sub-layer's output, a `Deferred` (normed before it is added) or a `DeferredMean` of at most two; one
        kernel does all of it. `lowered` [T, dim] in the run's type receives the new x as matrix products read it."""
        if x.dtype != torch.float32:
            raise ValueError("a norm after the sum runs over a 32-bit residual stream")
        factor, parts = 1.0, (pending,)
        if isinstance(pending, DeferredMean):
            factor, parts = pending.factor, tuple(pending.parts)
        if not 1 <= len(parts) <= 2:
            raise ValueError("a norm after the sum takes one or two pending outputs")
        values, weights, eps = [], [], set()
        for part in parts:
            if isinstance(part, Deferred):
                values.append(part.value); weights.append(part.weight); eps.add(float(part.eps))
            else:
                values.append(part); weights.append(None)
        if len(eps) > 1:
            raise ValueError("pending outputs that are normed share one eps")
        values += [None] * (2 - len(values)); weights += [None] * (2 - len(weights))
        ops.scaled_add_rmsnorm(x, values[0], weights[0], values[1], weights[1], eps.pop() if eps else 0.0, factor, alpha,
                               self.weight, self.eps, lowered, run_dtype=self.runtime.dtype)
        return x

    def add_normed(self, x: torch.Tensor, value: torch.Tensor, scale: float = 1.0, lowered: torch.Tensor | None = None) -> torch.Tensor:
        """The norm of a sub-layer's output alone, over a 32-bit stream and in place: x <- x + scale * norm(value), one
        kernel. `lowered` [T, dim] in the run's type receives the new x as matrix products read it."""
        if x.dtype != torch.float32:
            raise ValueError("a normed output joins a 32-bit residual stream")
        ops.residual_rmsnorm(x, value, self.weight, self.eps, None, None, 0.0, lowered, delta_scale=scale)
        return x

    @staticmethod
    def add(x: torch.Tensor, delta, extra: torch.Tensor | None = None) -> torch.Tensor:
        """x += delta (normed first if it is a `Deferred`) (+ extra), no norm of the sum: the stream itself."""
        value, weight, eps = (delta.value, delta.weight, delta.eps) if isinstance(delta, Deferred) else (delta, None, 0.0)
        if value is not None or extra is not None:
            ops.residual_rmsnorm(x, value, weight, eps, extra, None, 0.0, None)
        return x


@register_norm("layernorm")
class LayerNorm(Part):
    """y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias over a 32-bit residual stream.

    params: dim, eps, weight, bias (tensor names relative to the prefix; bias may be None).
    `forward(x, delta)` first adds what has not joined the stream yet: `delta` is None, one tensor, or a
    pair of tensors (the two sub-layers of a parallel block, either of which may be None), added as
    x + (a + b) in 32-bit in the same kernel as the norm. The stream must be float32 (a model with
    `residual_dtype="float32"`); the output is in the run's type, rounded once."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("dim", "eps", "weight")
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.weight_name = prefix + params["weight"]
        self.bias_name = prefix + params["bias"] if params.get("bias") else None
        self.weight = self.bias = None

    def tensor_specs(self):
        specs = [TensorSpec(self.weight_name, (self.dim,), kind="vector", init="ones")]
        if self.bias_name:
            specs.append(TensorSpec(self.bias_name, (self.dim,), kind="vector"))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]
        self.bias = tensors[self.bias_name] if self.bias_name else None

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    @staticmethod
    def _pair(delta):
        if isinstance(delta, Deferred):
            raise ValueError("layernorm: a sub-layer output that is normed before it is added needs an RMSNorm after it")
        if isinstance(delta, (tuple, list)):
            if len(delta) != 2:
                raise ValueError("layernorm adds at most two pending outputs at once")
            return delta[0], delta[1]
        return delta, None

    def forward(self, x: torch.Tensor, delta, rows: torch.Tensor | None = None,
                extra: torch.Tensor | None = None) -> torch.Tensor:
        if x.dtype != torch.float32:
            raise ValueError("layernorm runs over a 32-bit residual stream")
        if extra is not None:
            raise ValueError("layernorm takes no extra summand")
        first, second = self._pair(delta)
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.dim), dtype=self.runtime.dtype, device=x.device)
        return ops.residual_layernorm(x, first, second, self.weight, self.bias, self.eps, out, rows)

    @classmethod
    def add(cls, x: torch.Tensor, delta, extra: torch.Tensor | None = None) -> torch.Tensor:
        """x += the pending outputs, no norm: the stream itself."""
        first, second = cls._pair(delta)
        if first is not None or second is not None:
            ops.residual_layernorm(x, first, second, None, None, 0.0, None)
        return x
