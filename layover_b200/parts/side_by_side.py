"""Mixers that run side by side on the same input."""

from __future__ import annotations

from ..weights.loader import TensorSpec
from .base import Part, build_part, register_mixer
from .norm import Deferred, DeferredMean


@register_mixer("side_by_side")
class SideBySide(Part):
    """Several mixers read the same input; the result is the mean of their outputs, each RMS-normed over the model
    width with a weight of its own first: (1 / n) sum_i w_i * m_i(h) * rsqrt(mean(m_i(h)^2) + eps).

    The mean is not computed here: the outputs are handed on as a `DeferredMean`, and the norm of the stream that
    follows norms each, averages, adds and norms the sum in one kernel (a block whose norm comes after the sum).
    Each mixer keeps a cache or state of its own: `cache_need()` is the tuple of theirs and the cache view that
    `forward` receives has one view per mixer in `parts`.

    params: hidden, eps, mixers (a list of (mixer PartSpec, tensor-name prefix below this part's prefix, name of
    its output-norm weight relative to this part's prefix))."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "eps", "mixers")
        self.hidden, self.eps = int(params["hidden"]), float(params["eps"])
        self.mixers, self.weight_names = [], []
        for spec, sub_prefix, weight in params["mixers"]:
            self.mixers.append(build_part("mixer", spec, prefix + sub_prefix))
            self.weight_names.append(prefix + weight)
        if not self.mixers:
            raise ValueError("side_by_side: at least one mixer")
        self.weights = None

    def parts(self):
        return list(self.mixers)

    def tensor_specs(self):
        specs = [spec for mixer in self.mixers for spec in mixer.tensor_specs()]
        return specs + [TensorSpec(name, (self.hidden,), kind="vector", init="ones") for name in self.weight_names]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for mixer in self.mixers:
            mixer.bind(tensors, runtime)
        self.weights = [tensors[name] for name in self.weight_names]

    def cache_need(self):
        return tuple(mixer.cache_need() for mixer in self.mixers)

    def forward(self, h, batch, cache):
        outputs = [mixer.forward(h, batch, view) for mixer, view in zip(self.mixers, cache.parts)]
        return DeferredMean(tuple(Deferred(o, w, self.eps) for o, w in zip(outputs, self.weights)), 1.0 / len(outputs))
