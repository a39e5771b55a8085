"""Arrangements of a layer's parts."""

from __future__ import annotations

import contextlib

from .. import profiling
from .base import Part, build_part, register_block

_NO_RANGE = contextlib.nullcontext()


@register_block("pre_norm")
class PreNormBlock(Part):
    """x = x + mixer(norm(x)); x = x + feed_forward(norm(x)) (layover/model.py:164-166,224).

    The additions are not launched here: each sub-layer's output is handed on as `delta` and the
    next norm (of this block, of the next block, or the model's final norm) adds it into the
    residual stream before normalising.

    params: input_norm, mixer, post_norm, feed_forward (PartSpecs)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("input_norm", "mixer", "post_norm", "feed_forward")
        self.input_norm = build_part("norm", params["input_norm"], prefix)
        self.mixer = build_part("mixer", params["mixer"], prefix)
        self.post_norm = build_part("norm", params["post_norm"], prefix)
        self.feed_forward = build_part("feed_forward", params["feed_forward"], prefix)

    def parts(self):
        return [self.input_norm, self.mixer, self.post_norm, self.feed_forward]

    def tensor_specs(self):
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for part in self.parts():
            part.bind(tensors, runtime)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, delta, batch, cache, extra=None):
        if profiling.active():
            with profiling.nvtx_range("mixer"):
                h = self.input_norm.forward(x, delta, extra=extra)
                attended = self.mixer.forward(h, batch, cache)
            with profiling.nvtx_range("feed_forward"):
                h = self.post_norm.forward(x, attended)
                return x, self.feed_forward.forward(h)
        h = self.input_norm.forward(x, delta, extra=extra)
        attended = self.mixer.forward(h, batch, cache)
        h = self.post_norm.forward(x, attended)
        return x, self.feed_forward.forward(h)


@register_block("sandwich_norm")
class SandwichNormBlock(Part):
    """A norm before AND after each sub-layer: x = x + mixer_out_norm(mixer(input_norm(x))), then, where
    the layer has a feed-forward, x = x + ff_out_norm(feed_forward(post_norm(x))).

    As in the pre-norm block nothing is added here: a sub-layer's output is handed on as
    `norm.defer(output)` and the next norm of the stream (this block's, the next block's or the
    model's final one) norms it, adds it and norms the sum in one kernel.

    params: input_norm, mixer, mixer_out_norm (PartSpecs); post_norm, feed_forward, ff_out_norm
    (PartSpecs, or all three None for a layer without a feed-forward)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("input_norm", "mixer", "mixer_out_norm")
        self.input_norm = build_part("norm", params["input_norm"], prefix)
        self.mixer = build_part("mixer", params["mixer"], prefix)
        self.mixer_out_norm = build_part("norm", params["mixer_out_norm"], prefix)
        second = [params.get(k) for k in ("post_norm", "feed_forward", "ff_out_norm")]
        if any(p is None for p in second) and any(p is not None for p in second):
            raise ValueError("sandwich_norm: post_norm, feed_forward and ff_out_norm come together or not at all")
        self.post_norm = build_part("norm", second[0], prefix)
        self.feed_forward = build_part("feed_forward", second[1], prefix)
        self.ff_out_norm = build_part("norm", second[2], prefix)

    def parts(self):
        return [p for p in (self.input_norm, self.mixer, self.mixer_out_norm, self.post_norm, self.feed_forward,
                            self.ff_out_norm) if p is not None]

    def tensor_specs(self):
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for part in self.parts():
            part.bind(tensors, runtime)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, delta, batch, cache, extra=None):
        with profiling.nvtx_range("mixer") if profiling.active() else _NO_RANGE:
            h = self.input_norm.forward(x, delta, extra=extra)
            mixed = self.mixer_out_norm.defer(self.mixer.forward(h, batch, cache))
        if self.feed_forward is None:
            return x, mixed
        with profiling.nvtx_range("feed_forward") if profiling.active() else _NO_RANGE:
            h = self.post_norm.forward(x, mixed)
            return x, self.ff_out_norm.defer(self.feed_forward.forward(h))


@register_block("parallel")
class ParallelBlock(Part):
    """One norm, and both sub-layers read its output: h = norm(x); x = x + (mixer(h) + feed_forward(h)).

    Nothing is added here: the two outputs are handed on as a pair and the next norm of the stream
    (the next block's, or the model's final one) adds them, x + (a + b), in the kernel that norms the
    sum. A layer without a feed-forward hands on (a, None).

    params: input_norm, mixer (PartSpecs); feed_forward (a PartSpec or None)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("input_norm", "mixer")
        self.input_norm = build_part("norm", params["input_norm"], prefix)
        self.mixer = build_part("mixer", params["mixer"], prefix)
        self.feed_forward = build_part("feed_forward", params.get("feed_forward"), prefix)

    def parts(self):
        return [p for p in (self.input_norm, self.mixer, self.feed_forward) if p is not None]

    def tensor_specs(self):
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for part in self.parts():
            part.bind(tensors, runtime)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, delta, batch, cache, extra=None):
        h = self.input_norm.forward(x, delta, extra=extra)
        with profiling.nvtx_range("mixer") if profiling.active() else _NO_RANGE:
            mixed = self.mixer.forward(h, batch, cache)
        if self.feed_forward is None:
            return x, (mixed, None)
        with profiling.nvtx_range("feed_forward") if profiling.active() else _NO_RANGE:
            return x, (mixed, self.feed_forward.forward(h))


@register_block("post_norm")
class PostNormBlock(Part):
    """The norm comes after the sum, and the normed sum IS the stream: x = norm1(alpha * x + mixer(x)), then, where
    the layer has a feed-forward, x = norm2(alpha * x + feed_forward(x)). The sub-layers read the stream itself.

    The stream is 32-bit; each norm is one kernel that scales, adds (a mixer of several mixers hands over its
    outputs still to be normed and averaged: `DeferredMean`), norms and writes the stream back together with its
    copy in the run's type, which is what the next sub-layer's matrix products read (`batch.shared` carries that
    copy to the next block; a 32-bit run reads the stream directly). Nothing is pending when the block is done.

    params: mixer, mixer_norm (PartSpecs), alpha; feed_forward, ff_norm (PartSpecs, or both None)."""

    LOWERED = "post_norm.lowered_stream"

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("mixer", "mixer_norm")
        self.alpha = float(params.get("alpha", 1.0))
        self.mixer = build_part("mixer", params["mixer"], prefix)
        self.mixer_norm = build_part("norm", params["mixer_norm"], prefix)
        if (params.get("feed_forward") is None) != (params.get("ff_norm") is None):
            raise ValueError("post_norm: feed_forward and ff_norm come together or not at all")
        self.feed_forward = build_part("feed_forward", params.get("feed_forward"), prefix)
        self.ff_norm = build_part("norm", params.get("ff_norm"), prefix)

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ff_norm) if p is not None]

    def tensor_specs(self):
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for part in self.parts():
            part.bind(tensors, runtime)

    def cache_need(self):
        return self.mixer.cache_need()

    def _lowered(self, x, batch):
        """The stream in the run's type: what the block before left, else (the first block) a copy made now."""
        if self.runtime.dtype == x.dtype:
            return x, None
        held = batch.shared.get(self.LOWERED)
        if held is None or held[0] is not x:
            import torch
            from .. import ops
            lowered = torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device)
            ops.lower_rows(x, lowered)
            held = batch.shared[self.LOWERED] = (x, lowered)
        return held[1], held[1]

    def forward(self, x, delta, batch, cache, extra=None):
        if delta is not None or extra is not None:
            raise ValueError("post_norm: nothing can be pending when the block starts")
        h, lowered = self._lowered(x, batch)
        with profiling.nvtx_range("mixer") if profiling.active() else _NO_RANGE:
            self.mixer_norm.forward_after(x, self.mixer.forward(h, batch, cache), self.alpha, lowered)
        if self.feed_forward is not None:
            with profiling.nvtx_range("feed_forward") if profiling.active() else _NO_RANGE:
                self.ff_norm.forward_after(x, self.feed_forward.forward(h), self.alpha, lowered)
        return x, None


@register_block("output_norm")
class OutputNormBlock(PostNormBlock):
    """The norm sits on a sub-layer's OUTPUT only, and the normed output joins the stream times a constant:
    x = x + mult * norm1(mixer(x)), then, where the layer has a feed-forward, x = x + mult * norm2(feed_forward(x)).
    The sub-layers read the stream itself; the stream is never normed inside a layer.

    The stream is 32-bit; each sum is one kernel that norms the output, scales it, adds it and writes the stream's
    copy in the run's type for the next sub-layer's matrix products (`batch.shared` carries that copy to the next
    block; a 32-bit run reads the stream directly). Nothing is pending when the block is done.

    params: mixer, mixer_norm (PartSpecs), mult; feed_forward, ff_norm (PartSpecs, or both None)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.mult = float(params.get("mult", 1.0))

    def forward(self, x, delta, batch, cache, extra=None):
        if delta is not None or extra is not None:
            raise ValueError("output_norm: nothing can be pending when the block starts")
        h, lowered = self._lowered(x, batch)
        with profiling.nvtx_range("mixer") if profiling.active() else _NO_RANGE:
            self.mixer_norm.add_normed(x, self.mixer.forward(h, batch, cache), self.mult, lowered)
        if self.feed_forward is not None:
            with profiling.nvtx_range("feed_forward") if profiling.active() else _NO_RANGE:
                self.ff_norm.add_normed(x, self.feed_forward.forward(h), self.mult, lowered)
        return x, None
