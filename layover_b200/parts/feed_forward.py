"""Feed-forward parts."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, build_part, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    """down(act(gate(x)) * up(x)) without bias (layover/model.py:145-153); act = silu or relu.

    params: hidden, inter, activation ("silu", the default, or "relu"), gate, up, down (tensor names relative to the
    prefix). gate and up are stacked at load into one [2 inter, hidden] matrix so that one
    product reads x once. In a bfloat16 run whose width allows it, the rows are interleaved for
    the tensor-core product with the activation in its epilogue and no [T, 2 inter] tensor is ever
    written; otherwise the activation kernel reads both halves of its row. The product's epilogue
    knows silu only: with relu the interleaved product is followed by the activation kernel."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "inter", "gate", "up", "down")
        self.hidden, self.inter = int(params["hidden"]), int(params["inter"])
        self.activation = params.get("activation", "silu")
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"gated_mlp: unsupported activation {self.activation!r}")
        self.names = {k: prefix + params[k] for k in ("gate", "up", "down")}
        self.gate_up = self.down = None

    def tensor_specs(self):
        return [
            TensorSpec(self.names["gate"], (self.inter, self.hidden)),
            TensorSpec(self.names["up"], (self.inter, self.hidden)),
            TensorSpec(self.names["down"], (self.hidden, self.inter)),
        ]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        gate, up = tensors.pop(self.names["gate"]), tensors.pop(self.names["up"])
        self.fused = runtime.dtype == torch.bfloat16 and self.inter % ops.SWIGLU_BLOCK == 0
        if self.fused:
            self.gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.gate_up = torch.cat((gate, up), dim=0).contiguous()
        self.down = tensors[self.names["down"]]

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def activated(self, h: torch.Tensor) -> torch.Tensor:
        """silu(h Wg^T) * (h Wu^T) over the interleaved weights. Many tokens, or at most 16: one
        product with the activation in its epilogue. In between: product, then the activation kernel,
        which is faster there (a whole feed-forward at 64 tokens: 41.7 us against 43.5 us fused)."""
        tokens = h.shape[0]
        out = torch.empty((tokens, self.inter), dtype=torch.bfloat16, device=h.device)
        if self.activation == "silu" and (tokens > 128 or tokens <= 16) and ops.gemm_tcgen05_supports(h, self.gate_up):
            return ops.gemm_tcgen05(h, self.gate_up, out, epilogue="swiglu")
        gate_up = self.runtime.linear(h, self.gate_up)
        if self.activation == "silu":
            return ops.swiglu(gate_up, out, block=ops.SWIGLU_BLOCK)
        return ops.gated_act(gate_up, out, self.activation, block=ops.SWIGLU_BLOCK)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return self.runtime.linear(self.activated(h), self.down)
        gate_up = self.runtime.linear(h, self.gate_up)
        act = torch.empty((h.shape[0], self.inter), dtype=h.dtype, device=h.device)
        if self.activation == "silu":
            ops.swiglu(gate_up, act)
        else:
            ops.gated_act(gate_up, act, self.activation)
        return self.runtime.linear(act, self.down)


@register_feed_forward("mlp")
class MLP(Part):
    """down(act(up(x))) without gate and without bias; act = "relu2" (the square of relu), "gelu_tanh" or "silu".

    params: hidden, inter, activation (default "relu2"), up, down (tensor names relative to the prefix)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "inter", "up", "down")
        self.hidden, self.inter = int(params["hidden"]), int(params["inter"])
        self.activation = params.get("activation", "relu2")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"mlp: unsupported activation {self.activation!r}")
        self.names = {k: prefix + params[k] for k in ("up", "down")}
        self.up = self.down = None

    def tensor_specs(self):
        return [TensorSpec(self.names["up"], (self.inter, self.hidden)),
                TensorSpec(self.names["down"], (self.hidden, self.inter))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.up, self.down = tensors[self.names["up"]], tensors[self.names["down"]]

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        up = self.runtime.linear(h, self.up)
        return self.runtime.linear(ops.activation(up, up, self.activation), self.down)


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    """A mixture of small gated feed-forwards: every token goes to the `top` experts with the largest router
    scores and their outputs are added; optionally a shared expert that every token uses is added too.

        z = router h (32-bit), s = sigmoid(z); chosen = the `top` largest; no renormalisation of the chosen scores
        out = sum over chosen e of expert_e(s_e h) + sigmoid(shared_gate . h) * shared(h)
        expert(x) = down(act(gate x) * (up x)), act = silu (or relu)

    The score scales the expert's INPUT (`weight_on` = "input"), or, with `weight_on` = "output", its output:
    out = sum over chosen e of s_e expert_e(h). Experts without a gate (`gated` False): expert(x) = down(relu(up x)^2)
    (`activation` "relu2"; there is no expert_gate tensor). The choice may be made on corrected scores (`correction`: a
    tensor of one number per expert, added to the sigmoids for the choice only), limited to the `keep_groups` best of
    `groups` equal groups of neighbouring experts (a group's score: the sum of its two largest corrected scores), and the
    chosen scores may be divided by their sum (`renormalize`) and multiplied by `route_scale`. On the device:
    route (one warp per token) -> group the (token, expert) pairs by expert -> one launch for all experts'
    gate/up products with the activation in its epilogue -> one for their down products -> the sum over a
    token's experts with the shared expert in the same kernel. Nothing comes back to the host in between,
    so a step with routed layers is captured in a CUDA graph like any other.

    The router is a kernel of its own (a warp's 32-bit dot product per logit); for many tokens in a bfloat16 run
    whose router weights are bfloat16 numbers it is the run's tensor-core product with 32-bit output, which is the
    same arithmetic, followed by the selection kernel.

    Two forms of the products. Few pairs (decode steps), and every float32 run: FFMA kernels that gather the
    rows by index, take the score into the 32-bit sums and stream each chosen expert's weights once. Many
    pairs in a bfloat16 run: the pairs' rows, scaled by their scores, are laid out expert by expert in tiles
    of 128 rows (each expert's group padded to whole tiles), and both products run on the tensor cores as
    ONE grouped launch each, a tile's weights chosen by a list that the grouping kernel leaves on the device;
    tiles without pairs are skipped.

    params: hidden, experts, top, inter, activation ("silu"), router (tensor name), expert_gate / expert_up /
    expert_down (tensor names with `{}` for the expert's index), shared (a feed-forward PartSpec or None),
    shared_gate (tensor name of a [1, hidden] matrix, or None: the shared expert is added as it is); optional gated,
    weight_on, correction (tensor name), groups, keep_groups, renormalize, route_scale."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.gated = bool(p.get("gated", True))
        self.require("hidden", "experts", "top", "inter", "router", "expert_up", "expert_down", *(["expert_gate"] if self.gated else []))
        self.hidden, self.experts, self.top, self.inter = (int(p[k]) for k in ("hidden", "experts", "top", "inter"))
        if not 0 < self.top <= self.experts:
            raise ValueError(f"routed_experts: top ({self.top}) must lie in 1..experts ({self.experts})")
        self.activation = p.get("activation", "silu")
        if self.activation not in ops.EXPERT_ACTIVATIONS:
            raise ValueError(f"routed_experts: unsupported activation {self.activation!r}")
        self.weight_on = p.get("weight_on", "input")
        if self.weight_on not in ("input", "output") or p.get("score", "sigmoid") != "sigmoid":
            raise ValueError("routed_experts: built for sigmoid scores that scale the expert's input or its output")
        if self.gated and self.activation == "relu2":
            raise ValueError("routed_experts: gated experts are built with silu or relu")
        if not self.gated and (self.activation != "relu2" or self.weight_on != "output"):
            raise ValueError("routed_experts: experts without a gate are built with the squared relu and weights on their outputs")
        self.renormalize, self.route_scale = bool(p.get("renormalize", False)), float(p.get("route_scale", 1.0))
        self.groups = int(p.get("groups") or 0)
        self.keep_groups = int(p.get("keep_groups") or self.groups)
        if self.groups > 1 and (self.experts % self.groups or not 0 < self.keep_groups <= self.groups
                                or self.keep_groups * (self.experts // self.groups) < self.top):
            raise ValueError(f"routed_experts: {self.experts} experts in {self.groups} groups of which {self.keep_groups} are kept "
                             f"cannot give a token {self.top} experts")
        self.correction_name = prefix + p["correction"] if p.get("correction") else None
        self.router_name = prefix + p["router"]
        kinds = ("gate", "up", "down") if self.gated else ("up", "down")
        self.expert_names = [{k: prefix + p["expert_" + k].format(e) for k in kinds} for e in range(self.experts)]
        self.shared = build_part("feed_forward", p.get("shared"), prefix)
        self.shared_gate_name = prefix + p["shared_gate"] if p.get("shared_gate") else None
        if self.shared_gate_name and self.shared is None:
            raise ValueError("routed_experts: a shared gate without a shared expert")
        self.router = self.gate_up = self.down = self.shared_gate = self.correction = None

    def parts(self):
        return [self.shared] if self.shared is not None else []

    def tensor_specs(self):
        specs = [TensorSpec(self.router_name, (self.experts, self.hidden), kind="keep32")]
        if self.correction_name:
            specs.append(TensorSpec(self.correction_name, (self.experts,), kind="keep32"))
        for names in self.expert_names:
            if self.gated:
                specs.append(TensorSpec(names["gate"], (self.inter, self.hidden)))
            specs += [TensorSpec(names["up"], (self.inter, self.hidden)), TensorSpec(names["down"], (self.hidden, self.inter))]
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        if self.shared_gate_name:
            specs.append(TensorSpec(self.shared_gate_name, (1, self.hidden), kind="keep32"))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.router = tensors[self.router_name]
        self.correction = tensors[self.correction_name] if self.correction_name else None
        self._route = dict(correction=self.correction, groups=self.groups, keep_groups=self.keep_groups,
                           renormalize=self.renormalize, route_scale=self.route_scale)
        # one copy of the experts' weights serves both forms: where the tensor-core product can fuse the activation
        # (bfloat16, silu, widths in blocks of 64) every expert's gate and up rows are interleaved for it
        self.interleaved = (self.gated and runtime.dtype == torch.bfloat16 and self.activation == "silu"
                            and self.inter % ops.SWIGLU_BLOCK == 0)
        stack = ops.interleave_gate_up if self.interleaved else (lambda gate, up: torch.cat((gate, up), dim=0))
        if self.gated:
            self.gate_up = torch.stack([stack(tensors.pop(n["gate"]), tensors.pop(n["up"])) for n in self.expert_names]).contiguous()
        else:       # experts without a gate: [experts, inter, hidden]
            self.gate_up = torch.stack([tensors.pop(n["up"]) for n in self.expert_names]).contiguous()
        self.down = torch.stack([tensors.pop(n["down"]) for n in self.expert_names]).contiguous()
        self.grouped = (runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0
                        and ops.gemm_tcgen05_supports(self.gate_up.view(-1, self.hidden), self.down.view(-1, self.inter)))
        if self.shared is not None:
            self.shared.bind(tensors, runtime)
        self.shared_gate = tensors[self.shared_gate_name].reshape(-1).contiguous() if self.shared_gate_name else None
        # In a bfloat16 run whose router weights are bfloat16 numbers, the logits of many tokens are one tensor-core
        # product: bfloat16 x bfloat16 is exact in 32-bit and the sums are 32-bit, so these are 32-bit logits.
        self.router_matrix = None
        if runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0:
            rows = [self.router] + ([self.shared_gate[None]] if self.shared_gate is not None else [])
            stacked = torch.cat(rows, dim=0)
            if bool((stacked.to(torch.bfloat16).float() == stacked).all()):
                padded = torch.zeros((-(-stacked.shape[0] // 8) * 8, self.hidden), dtype=torch.bfloat16, device=stacked.device)
                padded[: stacked.shape[0]] = stacked.to(torch.bfloat16)
                self.router_matrix = padded

    def kernel_libraries(self, dtype):
        return ("elementwise", "moe") + (("gemm_tcgen05",) if dtype == torch.bfloat16 else ())

    def route(self, h: torch.Tensor):
        """(expert ids [T, top] int32, their scores [T, top] float32, the shared expert's factor [T] or None)."""
        tokens = h.shape[0]
        ids = torch.empty((tokens, self.top), dtype=torch.int32, device=h.device)
        scores = torch.empty((tokens, self.top), dtype=torch.float32, device=h.device)
        factor = torch.empty((tokens,), dtype=torch.float32, device=h.device) if self.shared_gate is not None else None
        if self.router_matrix is not None and tokens > self.ROUTE_PRODUCT_FROM:
            logits = self.runtime.linear(h, self.router_matrix, out_dtype=torch.float32)
            ops.moe_select(logits, self.experts, self.top, ids, scores, factor, **self._route)
        else:
            ops.moe_route(h, self.router, self.top, ids, scores, self.shared_gate, factor, **self._route)
        return ids, scores, factor

    ROUTE_PRODUCT_FROM = 64 # tokens beyond which a bfloat16 run's router logits are a tensor-core product
    FEW_PER_EXPERT = 4      # up to this many pairs per expert on average the weight-streaming kernels run; beyond, in
                            # bfloat16, the grouped tensor-core products (in float32 the tiled FFMA kernel)

    def _forward_grouped(self, h, ids, scores, factor):
        tokens, pairs = h.shape[0], h.shape[0] * self.top
        rows = ops.moe_padded_rows(pairs, self.experts)
        tiles = rows // ops.MOE_TILE_ROWS
        place_of = torch.empty((pairs,), dtype=torch.int32, device=h.device)
        tile_up = torch.empty((tiles + 1,), dtype=torch.int32, device=h.device)      # the last entry: the tiles in use
        tile_down = torch.empty((tiles + 1,), dtype=torch.int32, device=h.device)
        on_input = self.weight_on == "input"
        up_rows = (2 if self.gated else 1) * self.inter
        ops.moe_group_tiles(ids, self.experts, place_of, tile_up, tile_down, up_rows, self.hidden)
        scaled = torch.empty((rows, self.hidden), dtype=h.dtype, device=h.device)
        ops.moe_scatter_rows(h, place_of, scores if on_input else None, scaled, self.top)
        act = torch.empty((rows, self.inter), dtype=h.dtype, device=h.device)
        weights = self.gate_up.view(self.experts * up_rows, self.hidden)
        if not self.gated:
            ops.gemm_tcgen05_grouped(scaled, weights, act, tile_up, self.experts)
            ops.activation(act, act, self.activation)
        elif self.interleaved:
            ops.gemm_tcgen05_grouped(scaled, weights, act, tile_up, self.experts, epilogue="swiglu")
        else:
            both = torch.empty((rows, 2 * self.inter), dtype=h.dtype, device=h.device)
            ops.gemm_tcgen05_grouped(scaled, weights, both, tile_up, self.experts)
            ops.gated_act(both, act, self.activation)
        y = torch.empty((rows, self.hidden), dtype=h.dtype, device=h.device)     # rounded like every product's output; summed in 32-bit
        ops.gemm_tcgen05_grouped(act, self.down.view(self.experts * self.hidden, self.inter), y, tile_down, self.experts)
        shared = self.shared.forward(h) if self.shared is not None else None
        out = torch.empty((tokens, self.hidden), dtype=h.dtype, device=h.device)
        return ops.moe_combine(y, out, self.top, None if on_input else scores, shared, factor, rows=place_of)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        tokens, pairs = h.shape[0], h.shape[0] * self.top
        ids, scores, factor = self.route(h)
        if self.grouped and pairs > self.FEW_PER_EXPERT * self.experts:
            return self._forward_grouped(h, ids, scores, factor)
        offsets = torch.empty((self.experts + 1,), dtype=torch.int32, device=h.device)
        order = torch.empty((pairs,), dtype=torch.int32, device=h.device)
        ops.moe_group(ids, self.experts, offsets, order)
        act = torch.empty((pairs, self.inter), dtype=h.dtype, device=h.device)
        on_input = self.weight_on == "input"
        ops.moe_expert_up(h, order, offsets, scores if on_input else None, self.gate_up, act, self.top, self.activation,
                          self.interleaved, self.gated)
        y = torch.empty((pairs, self.hidden), dtype=torch.float32, device=h.device)
        ops.moe_expert_down(act, order, offsets, self.down, y)
        shared = self.shared.forward(h) if self.shared is not None else None
        out = torch.empty((tokens, self.hidden), dtype=h.dtype, device=h.device)
        return ops.moe_combine(y, out, self.top, None if on_input else scores, shared, factor)
