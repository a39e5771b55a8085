"""Attention over a latent: the cache holds one small vector per token, and every head's keys and
values are linear maps of it."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import PagedKVNeed, Part, build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Part):
    """A token leaves c = rmsnorm(W_down h)[:rank] and one rotated key part k_r (`rot_dim` channels, shared by
    all heads) in the cache. Head h has queries [q_h: dim | q_r,h: rot_dim (rotated)], keys [W_uk,h c | k_r]
    and values W_uv,h c; causal softmax attention with a scale of its own (over every earlier token, or, with
    `window`, over the token itself and the window - 1 before it); the concatenated heads are multiplied channel by
    channel with sigmoid(W_g h) (where the layer has a W_g) and projected.

    The two maps are never applied to cached tokens. Since (W_uk,h c) . q_h = c . (W_uk,h^T q_h) and
    sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j, a step is attention with ONE key/value head whose key is the
    cache row [c | k_r], whose value is the row's first `rank` channels (the cache keeps one store, not two),
    and whose query of head h is [W_uk,h^T q_h | q_r,h]; the heads' outputs, still `rank` wide, then pass
    W_uv,h with the gate in the same kernel. A layer with `shares_cache` has no W_down: it reads the rows of
    an earlier layer (the schedule names it) through maps of its own.

    params: hidden, heads, head_dim (unrotated), rot_dim, v_head_dim, kv_rank, scale, norm_eps, position (a
    PartSpec over rot_dim channels whose table the kernel applies to neighbouring pairs), shares_cache; window (None:
    every earlier token) and cache_window (the window the cached rows are kept for: the widest of this layer's and of
    the layers' that read its rows; default: window); tensor names q, down, down_norm, up_k, up_v, o and gate (None:
    no gate) relative to the prefix.

    32-bit: the latent's norm, the rotation, scores, softmax and its weights (the tensor-core kernels run in
    their variant whose weights keep 16 bits of mantissa), the gate. The stacked projection leaves 32-bit rows
    in both precisions, and the fold W_uk,h^T q_h reads them unrounded."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "heads", "head_dim", "rot_dim", "v_head_dim", "kv_rank", "scale", "norm_eps", "position",
                     "q", "up_k", "up_v", "o")
        p = params
        self.hidden, self.heads, self.dim, self.rot, self.vdim, self.rank = (
            int(p[k]) for k in ("hidden", "heads", "head_dim", "rot_dim", "v_head_dim", "kv_rank"))
        self.scale, self.norm_eps = float(p["scale"]), float(p["norm_eps"])
        self.shares_cache = bool(p.get("shares_cache", False))
        if self.rot % 2 or self.rot < 0:
            raise ValueError(f"latent_attention: rot_dim must be even, got {self.rot}")
        self.row = self.rank + self.rot           # a cache row's channels in use
        if self.row > ops.ATTENTION_SIMT_MAX_DIM:
            raise ValueError(f"latent_attention: kv_rank + rot_dim up to {ops.ATTENTION_SIMT_MAX_DIM} is supported, got {self.row}")
        self.gated = bool(p.get("gate"))
        self.window = int(p["window"]) if p.get("window") else None
        self.cache_window = int(p["cache_window"]) if p.get("cache_window") else self.window
        if self.window is not None and (self.window < 1 or self.cache_window < self.window):
            raise ValueError("latent_attention: a window holds at least the token itself, and the cached rows are kept at least that long")
        wanted = ["q", "up_k", "up_v", "o"] + (["gate"] if self.gated else []) + ([] if self.shares_cache else ["down", "down_norm"])
        self.require(*wanted)
        self.names = {k: prefix + p[k] for k in wanted}
        self.position = build_part("position", p["position"], prefix)
        if getattr(self.position, "pairing", None) != "neighbours" or getattr(self.position, "rotated", None) != self.rot:
            raise ValueError("latent_attention: the position part must rotate neighbouring pairs over rot_dim channels")
        self.room = None          # once bound: a row's room in the cache (16s for the tensor-core kernels, else 4s)

    def tensor_specs(self):
        n = self.names
        specs = [TensorSpec(n["q"], (self.heads * (self.dim + self.rot), self.hidden))]
        if not self.shares_cache:
            specs += [TensorSpec(n["down"], (self.row, self.hidden)),
                      TensorSpec(n["down_norm"], (self.rank,), kind="vector", init="ones")]
        specs += [TensorSpec(n["up_k"], (self.heads * self.dim, self.rank)), TensorSpec(n["up_v"], (self.heads * self.vdim, self.rank))]
        if self.gated:
            specs.append(TensorSpec(n["gate"], (self.heads * self.vdim, self.hidden)))
        specs.append(TensorSpec(n["o"], (self.hidden, self.heads * self.vdim)))
        return specs + self.position.tensor_specs()

    def _decode_groups(self) -> int:
        """The heads as the fewest equal groups of at most 16: a group is the rows of one tile of the decode kernel."""
        return next(g for g in range(1, self.heads + 1) if self.heads % g == 0 and self.heads // g <= 16)

    def _on_tensor_cores(self, dtype) -> bool:
        return dtype == torch.bfloat16 and self.row <= 256      # a cache row is the tensor-core kernels' head

    def _room(self, dtype) -> int:
        step = 16 if self._on_tensor_cores(dtype) else 4
        return -(-self.row // step) * step

    def cache_need(self):
        room = self.room if self.room is not None else -(-self.row // 4) * 4
        return PagedKVNeed(1, room, window=self.cache_window, values_in_keys=True)

    def parts(self):
        return [self.position]

    def kernel_libraries(self, dtype):
        return ("elementwise", "latent", "attention_mma" if self._on_tensor_cores(dtype) else "attention_simt")

    def tile_sizes(self, dtype):
        return (ops.attention_mma_block_queries() if self._on_tensor_cores(dtype) else ops.attention_simt_block_queries(),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        rows = [tensors.pop(n["q"])] + ([tensors.pop(n["gate"])] if self.gated else [])
        if not self.shares_cache:
            rows.append(tensors.pop(n["down"]))
            self.down_norm = tensors[n["down_norm"]]
        used = sum(r.shape[0] for r in rows)
        if used % 16:           # whole 16-byte pieces per output row
            rows.append(torch.zeros((16 - used % 16, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()                    # [q | gate | down (| padding)]
        self.q_off, self.gate_off = 0, self.heads * (self.dim + self.rot)
        self.down_off = -1 if self.shares_cache else self.gate_off + (self.heads * self.vdim if self.gated else 0)
        # W_uk,h^T as the per-head product reads it: [heads, rank, dim]
        self.w_fold = tensors.pop(n["up_k"]).view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_up_v = tensors.pop(n["up_v"]).view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = tensors[n["o"]]
        self.position.bind(tensors, runtime)
        self.tensor_cores = self._on_tensor_cores(runtime.dtype)
        if self.tensor_cores:
            ops.attention_scratch(runtime.device)      # made now, never inside a graph capture
        self.room = self._room(runtime.dtype)

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        tokens, group, room = h.shape[0], batch.groups[cache.group], self.room
        proj = self.runtime.linear(h, self.w_in, out_dtype=torch.float32)
        table = self.position.tables(batch)
        q = torch.empty((tokens, self.heads * room), dtype=h.dtype, device=h.device)
        ops.latent_rows(proj, self.q_off, self.down_off, None if self.shares_cache else self.down_norm, self.norm_eps, table,
                        None if self.shares_cache else group.slot_map, None if self.shares_cache else cache.k_pool, q,
                        self.heads, self.dim, self.rot, self.rank, cache.page_tokens)
        q3 = q.view(tokens, self.heads, room)
        ops.heads_linear(proj[:, : self.heads * (self.dim + self.rot)].unflatten(1, (self.heads, self.dim + self.rot))[:, :, : self.dim],
                         self.w_fold, q3[:, :, : self.rank])
        out = torch.empty((tokens, self.heads * room), dtype=h.dtype, device=h.device)
        if self.tensor_cores:
            ops.attention_bf16(q, cache, out, group.block_table, batch, self.heads, 1, room, cache.page_tokens, self.scale,
                               self.window or 0, exact_weights=True, decode_share=self._decode_groups())
        else:
            ops.attention_f32(q, cache, out, group.block_table, batch, self.heads, 1, room, cache.page_tokens, self.scale,
                              self.window or 0, room)
        gated = torch.empty((tokens, self.heads * self.vdim), dtype=h.dtype, device=h.device)
        ops.heads_linear(out.view(tokens, self.heads, room)[:, :, : self.rank], self.w_up_v, gated.view(tokens, self.heads, self.vdim),
                         gate=proj[:, self.gate_off: self.gate_off + self.heads * self.vdim] if self.gated else None)
        return self.runtime.linear(gated, self.w_o)
