"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import math

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import PagedKVNeed, Part, PartSpec, build_part, register_mixer


@register_mixer("attention")
class Attention(Part):
    """q/k/v projections without bias, optional per-head RMSNorm of q and k, a position encoding,
    keys and values written to their pages, causal attention over the block table with scale
    1/sqrt(head_dim), output projection (layover/model.py:105-142).

    params: hidden, q_heads, kv_heads, head_dim; qk_norm_eps (None: no per-head norm);
    position (a PartSpec or None); window (None: every earlier key is seen);
    shares_cache (True: the layer has no k/v projections and attends over another layer's
    pages); tensor names q, k, v, o (and q_norm, k_norm with a per-head norm) relative to the
    prefix: the architecture's spec gives them, the part knows no checkpoint's naming.

    Kernels are chosen when the part is bound: a float32 run attends with the one 32-bit kernel
    for every segment length; a bfloat16 run with the tensor-core kernels (tcgen05 tiles where
    they take the head size, mma.sync tiles elsewhere, the split decode kernel for single
    tokens) and, for steps of few tokens, a q/k/v product with norm, rotation and page write in
    its epilogue.

    The three projections are stacked at load into one [(q_heads + 2 kv_heads) head_dim, hidden]
    matrix (the reference runs three products, layover/model.py:121-123).

    Further options, for other designs than the reference's: `scale` (instead of 1/sqrt(head_dim));
    `v_head_dim` (values of another size than keys); `qk_norm` = "whole" (ONE RMSNorm over the
    whole q projection and one over the whole k projection, all heads at once, with a weight per
    channel, instead of a norm per head); `sink` (tensor name: a learned score per query head that
    joins the softmax's denominator and nothing else); `gate` (tensor name of a [q_heads, hidden]
    matrix: head h's output is multiplied by sigmoid(gate h)_h before the output projection).
    Any of these makes the part take its general path: the gate's rows are stacked under q, k, v
    for one product, one kernel norms q and k over their whole rows, writes the pages and makes
    the gates, and the attention runs with sinks and gates as parameters of its kernels: in a float32
    run the 32-bit kernel; in a bfloat16 run the tensor-core kernels (tiles for prompt portions,
    the split kernel for single tokens) in their variant whose weights enter the second product with
    16 bits of mantissa, where the head sizes are multiples of 16 (keys and values of different
    sizes then share pages of the larger size, zero-filled: zeros change no score and no sum), and
    the 32-bit kernel on bfloat16 pages otherwise. That path has no shared cache.

    More options of the general path: `q_bias`, `k_bias`, `v_bias` (tensor names: a bias per channel of a
    projection, added before anything else); a `position` whose table rotates only the first channels of a
    head; `chunk` (a chunked mask: position i sees j <= i only where floor(i / chunk) == floor(j / chunk),
    chunks counted from position 0 of the sequence; the cache gives back the pages of finished chunks);
    `gate_kind` = "channel" (`gate` is then a [q_heads * v_head_dim, hidden] matrix and every channel of
    the concatenated heads is multiplied by its own sigmoid; default "head"); `value_blend` = "keep" (this
    layer's values, bias included, are kept for the rest of the step) or "blend" (the values that go to the
    cache are (1 - w) v + w kept values of the same token, w = the scalar tensor `value_blend_weight`).
    With any of these the stacked product leaves 32-bit rows and ONE kernel adds the biases, rotates, blends
    and writes q and the pages (rounded once); a channel gate is one more small kernel after the attention.
    They do not combine with the whole-row norm or head gates; a norm per head (`qk_norm_eps` with the default
    `qk_norm`) does: it is applied in the same kernel, after the biases and before the rotation.
    `values` = "keys": the layer has no v projection; what a key/value head stores as its value is its raw key
    projection, taken before the key is normed and turned (`v_head_dim` = `head_dim`). A `position` that pairs neighbouring channels (`rotary_pairs`) turns channels 2i
    and 2i + 1 together. Both take this path.
    `keep_first` (with `window`): the first `keep_first` tokens of a sequence stay visible behind the window, at
    their own positions; their pages stay in the cache. `exact_weights` = True asks for this path (32-bit
    projection rows, softmax weights that keep 16 bits of mantissa in the second product) without any other option."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "q_heads", "kv_heads", "head_dim")
        p = params
        self.hidden, self.q_heads, self.kv_heads, self.dim = (int(p[k]) for k in ("hidden", "q_heads", "kv_heads", "head_dim"))
        if self.q_heads % self.kv_heads:
            raise ValueError(f"q_heads ({self.q_heads}) must be divisible by kv_heads ({self.kv_heads})")
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.qk_norm = p.get("qk_norm", "per_head")
        if self.qk_norm not in ("per_head", "whole"):
            raise ValueError(f"qk_norm must be 'per_head' or 'whole', got {self.qk_norm!r}")
        self.biases = [k for k in ("q_bias", "k_bias", "v_bias") if p.get(k)]
        self.values_from_keys = p.get("values", "own") == "keys"
        if p.get("values", "own") not in ("own", "keys") or (self.values_from_keys and (self.vdim != self.dim or p.get("v_bias")
                                                                                      or p.get("value_blend") or p.get("shares_cache"))):
            raise ValueError("attention: values are 'own' or 'keys'; values that are the keys have the keys' size, no bias, no "
                             "blend and a cache of their own")
        self.chunk = int(p.get("chunk") or 0)
        self.gate_kind = p.get("gate_kind", "head")
        self.value_blend = p.get("value_blend")
        if self.gate_kind not in ("head", "channel") or self.value_blend not in (None, "keep", "blend"):
            raise ValueError("attention: gate_kind is 'head' or 'channel', value_blend None, 'keep' or 'blend'")
        position = p.get("position")
        partial = bool(position and (int(position.params.get("rotated") or p["head_dim"]) != int(p["head_dim"])
                                     or position.kind == "rotary_pairs"))
        # biases, a partial rotation, a blend of values or a gate per channel: one kernel over 32-bit projection rows
        self.keep_first = int(p.get("keep_first") or 0)
        if self.keep_first < 0 or (self.keep_first and not p.get("window")):
            raise ValueError("attention: keep_first is a number of tokens and comes with a window")
        self.rows32 = bool(self.biases or partial or self.value_blend or (p.get("gate") and self.gate_kind == "channel")
                           or (position and (p.get("v_head_dim") or p["head_dim"]) != p["head_dim"]) or self.chunk
                           or self.keep_first or p.get("exact_weights") or self.values_from_keys)
        self.general = bool(self.vdim != self.dim or self.qk_norm == "whole" or p.get("sink") or p.get("gate") or self.rows32)
        if self.general:
            if (self.dim % 4 or self.vdim % 4) and not self.rows32:
                raise ValueError(f"head sizes must be multiples of 4, got {self.dim} and {self.vdim}")
        elif self.dim % 16:
            raise ValueError(f"head_dim must be a multiple of 16, got {self.dim}")
        # the tensor-core kernels take head sizes up to 256; the path over 32-bit projection rows may use the 32-bit
        # attention kernel instead, which takes more
        if max(self.dim, self.vdim) > (ops.ATTENTION_SIMT_MAX_DIM if self.rows32 else 256):
            raise ValueError(f"head sizes up to {ops.ATTENTION_SIMT_MAX_DIM if self.rows32 else 256} are supported, got {max(self.dim, self.vdim)}")
        self.qk_norm_eps = p.get("qk_norm_eps")
        self.window = p.get("window")
        self.shares_cache = bool(p.get("shares_cache", False))
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.dim))
        self.position = build_part("position", p.get("position"), prefix)
        if self.general and (self.shares_cache or (self.position is not None and not self.rows32)):
            raise ValueError("attention with sinks, head gates, a whole-row norm or its own value size has no rotation "
                             "and no shared cache")
        if self.rows32 and ((self.qk_norm_eps is not None and self.qk_norm == "whole") or (p.get("gate") and self.gate_kind == "head")):
            raise ValueError("attention: biases, partial rotation, chunks, value blends and channel gates do not combine "
                             "with whole-row q/k norms or head gates")
        if self.chunk and self.window:
            raise ValueError("attention: a window and a chunked mask do not combine")
        if self.chunk < 0:
            raise ValueError("attention: chunk must be positive")
        wanted = ["q", "o"] + ([] if self.shares_cache else (["k"] if self.values_from_keys else ["k", "v"]))
        if self.qk_norm_eps is not None:
            wanted += ["q_norm"] + ([] if self.shares_cache else ["k_norm"])
        wanted += [k for k in ("sink", "gate") if p.get(k)] + self.biases
        if self.value_blend == "blend":
            wanted.append("value_blend_weight")
        self.require(*wanted)
        self.names = {k: prefix + p[k] for k in wanted}
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = self.sink = None
        self._attend = self._project_heads = None
        self.room = None        # once bound: the size keys, values and queries are padded to for the tensor-core kernels
        # where the tensor-core kernels do not run: the room of a key and of a value in their pages (the 32-bit kernel
        # reads four channels at a time; the kernel over 32-bit projection rows fills the rest of the room with zeros)
        self.k_room, self.v_room = (-(-self.dim // 4) * 4, -(-self.vdim // 4) * 4) if self.rows32 else (self.dim, self.vdim)

    # ---- what it wants
    def tensor_specs(self):
        n = self.names
        specs = [TensorSpec(n["q"], (self.q_heads * self.dim, self.hidden))]
        if not self.shares_cache:
            specs.append(TensorSpec(n["k"], (self.kv_heads * self.dim, self.hidden)))
            if not self.values_from_keys:
                specs.append(TensorSpec(n["v"], (self.kv_heads * self.vdim, self.hidden)))
        specs.append(TensorSpec(n["o"], (self.hidden, self.q_heads * self.vdim)))
        if self.qk_norm_eps is not None:
            whole = self.qk_norm == "whole"
            specs.append(TensorSpec(n["q_norm"], (self.q_heads * self.dim if whole else self.dim,), kind="vector", init="ones"))
            if not self.shares_cache:
                specs.append(TensorSpec(n["k_norm"], (self.kv_heads * self.dim if whole else self.dim,), kind="vector",
                                        init="ones"))
        if "sink" in n:
            specs.append(TensorSpec(n["sink"], (self.q_heads,), kind="vector"))
        if "gate" in n:
            specs.append(TensorSpec(n["gate"], (self.q_heads * (self.vdim if self.gate_kind == "channel" else 1), self.hidden)))
        sizes = {"q_bias": self.q_heads * self.dim, "k_bias": self.kv_heads * self.dim, "v_bias": self.kv_heads * self.vdim}
        specs += [TensorSpec(n[k], (sizes[k],), kind="vector") for k in self.biases]
        if self.value_blend == "blend":
            specs.append(TensorSpec(n["value_blend_weight"], (), kind="vector"))
        if self.position is not None:
            specs += self.position.tensor_specs()
        return specs

    def cache_need(self):
        chunk = self.chunk or None
        if self.room is not None:
            return PagedKVNeed(self.kv_heads, self.room, self.window, chunk=chunk, keep_first=self.keep_first)
        return PagedKVNeed(self.kv_heads, self.k_room, self.window, self.v_room if self.v_room != self.k_room else None, chunk=chunk,
                           keep_first=self.keep_first)

    def _on_tensor_cores(self, dtype) -> bool:
        """Whether the general path runs on the tensor-core kernels in a run of `dtype`."""
        return (self.general and dtype == torch.bfloat16 and self.q_heads // self.kv_heads <= 16 and max(self.dim, self.vdim) <= 256
                and (self.rows32 or (self.dim % 16 == 0 and self.vdim % 16 == 0)))     # rows32: any size, padded to 16s

    def parts(self):
        return [self.position] if self.position is not None else []

    def kernel_libraries(self, dtype):
        if self._on_tensor_cores(dtype):
            return ("elementwise", "attention_mma")
        if dtype == torch.float32 or self.general:
            return ("elementwise", "attention_simt")
        names = ["elementwise", "attention_mma"]
        if ops.attention_tcgen05_takes_heads(self.q_heads, self.kv_heads, self.dim):
            names.append("attention_tcgen05")
        return tuple(names)

    def tile_sizes(self, dtype):
        if self._on_tensor_cores(dtype):
            return (ops.attention_mma_block_queries(),)
        if dtype == torch.float32 or self.general:
            return (ops.attention_simt_block_queries(),)
        sizes = [ops.attention_mma_block_queries()]
        if ops.attention_tcgen05_takes_heads(self.q_heads, self.kv_heads, self.dim):
            sizes.append(ops.TCGEN05_TILE)
        return tuple(sizes)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        if self.general:
            return self._bind_general(tensors, runtime)
        if runtime.dtype == torch.float32:
            self._attend, self._project_heads = ops.attention_f32, None
        else:
            ops.attention_scratch(runtime.device)      # made now, never inside a graph capture
            self._attend, self._project_heads = ops.attention_bf16, ops.gemm_qkv_heads
        n = self.names
        if self.shares_cache:
            self.w_qkv = tensors[n["q"]]
        else:
            self.w_qkv = torch.cat((tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"])), dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.qk_norm_eps is not None:
            self.q_norm_w = tensors[n["q_norm"]]
            self.k_norm_w = None if self.shares_cache else tensors[n["k_norm"]]
        if self.position is not None:
            self.position.bind(tensors, runtime)

    def _bind_general(self, tensors, runtime):
        n = self.names
        rows = [tensors.pop(n["q"]), tensors.pop(n["k"])] + ([] if self.values_from_keys else [tensors.pop(n["v"])])
        if "gate" in n:
            rows.append(tensors.pop(n["gate"]))
        used = sum(r.shape[0] for r in rows)
        if used % 16:           # whole 16-byte pieces per output row, whatever the head counts
            rows.append(torch.zeros((16 - used % 16, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.qk_norm_eps is not None:
            self.q_norm_w, self.k_norm_w = tensors[n["q_norm"]], tensors[n["k_norm"]]
        self.sink = tensors[n["sink"]] if "sink" in n else None
        self.bias = {k: tensors[n[k]] for k in self.biases}
        self.blend_weight = tensors[n["value_blend_weight"]].reshape(1) if self.value_blend == "blend" else None
        if self.position is not None:
            self.position.bind(tensors, runtime)
        if self._on_tensor_cores(runtime.dtype):
            ops.attention_scratch(runtime.device)      # made now, never inside a graph capture
            self.room = -(-max(self.dim, self.vdim) // 16) * 16
        # the heads' outputs arrive padded: zero columns in the output matrix (a channel gate writes them dense)
        out_room = self.room or self.v_room
        if out_room != self.vdim and not ("gate" in n and self.gate_kind == "channel"):
            wide = torch.zeros((self.hidden, self.q_heads, out_room), dtype=self.w_o.dtype, device=self.w_o.device)
            wide[:, :, : self.vdim] = self.w_o.view(self.hidden, self.q_heads, self.vdim)
            self.w_o = wide.view(self.hidden, self.q_heads * out_room).contiguous()

    def _kept_values(self, batch, tokens, device):
        """The step's buffer of kept values [T, kv_heads * v_head_dim], 32-bit: made by the layer that keeps,
        found by the layers that blend (`batch.shared` lives for one step)."""
        key = ("value_blend", self.kv_heads, self.vdim)
        if self.value_blend == "keep":
            batch.shared[key] = torch.empty((tokens, self.kv_heads * self.vdim), dtype=torch.float32, device=device)
        elif key not in batch.shared:
            raise ValueError("attention: a layer blends its values before any layer of the model kept them")
        return batch.shared[key]

    def _forward_general(self, h, batch, cache):
        tokens, group = h.shape[0], batch.groups[cache.group]
        room = self.room or self.k_room
        q = torch.empty((tokens, self.q_heads * room), dtype=h.dtype, device=h.device)
        gates = None
        if self.rows32:
            proj = self.runtime.linear(h, self.w_qkv, out_dtype=torch.float32)
            table = self.position.tables(batch) if self.position is not None else None
            if self.position is not None and table is None:
                raise ValueError("attention: this position encoding offers no table for the fused kernel")
            blend = {None: 0, "keep": 1, "blend": 2}[self.value_blend]
            kept = self._kept_values(batch, tokens, h.device) if blend else None
            ops.heads_bias_rope_kv(proj, q, cache.k_pool, cache.v_pool, self.bias.get("q_bias"), self.bias.get("k_bias"),
                                   self.bias.get("v_bias"), table, group.slot_map, kept, blend, self.blend_weight,
                                   self.q_heads, self.kv_heads, self.dim, self.vdim, cache.page_tokens,
                                   self.q_norm_w, self.k_norm_w, float(self.qk_norm_eps or 0.0),
                                   neighbours=getattr(self.position, "pairing", "half") == "neighbours",
                                   values_from_keys=self.values_from_keys)
        else:
            proj = self.runtime.linear(h, self.w_qkv)
            if "gate" in self.names:
                gates = torch.empty((tokens, self.q_heads), dtype=torch.float32, device=h.device)
            ops.qk_rownorm_kv(proj, q, cache.k_pool, cache.v_pool, self.q_norm_w, self.k_norm_w, group.slot_map, gates,
                              self.q_heads, self.kv_heads, self.dim, self.vdim, cache.page_tokens, float(self.qk_norm_eps or 0.0))
        if self.room is not None:
            out = torch.empty((tokens, self.q_heads * room), dtype=h.dtype, device=h.device)
            ops.attention_bf16(q, cache, out, group.block_table, batch, self.q_heads, self.kv_heads, room, cache.page_tokens,
                               self.scale, self.window or 0, sinks=self.sink, gates=gates, exact_weights=True, chunk=self.chunk,
                               keep_first=self.keep_first)
        else:
            out = torch.empty((tokens, self.q_heads * self.v_room), dtype=h.dtype, device=h.device)
            ops.attention_f32(q, cache, out, group.block_table, batch, self.q_heads, self.kv_heads, self.k_room, cache.page_tokens,
                              self.scale, self.window or 0, self.v_room, self.sink, gates, chunk=self.chunk,
                              keep_first=self.keep_first)
        if self.rows32 and "gate" in self.names:
            at = self.q_heads * self.dim + self.kv_heads * (self.dim + (0 if self.values_from_keys else self.vdim))
            gated = torch.empty((tokens, self.q_heads * self.vdim), dtype=h.dtype, device=h.device)
            out = ops.channel_gate(out, proj[:, at: at + self.q_heads * self.vdim], gated, self.q_heads, self.vdim)
        return self.runtime.linear(out, self.w_o)

    # ---- one step
    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        if self.general:
            return self._forward_general(h, batch, cache)
        q = self.project(h, batch, cache)
        out = torch.empty_like(q)
        self.attend(q, cache, batch, batch.groups[cache.group], out)
        return self.runtime.linear(out, self.w_o)

    def project(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        """q [T, q_heads * head_dim], normed and rotated; this step's keys and values go to their pages."""
        tokens = h.shape[0]
        own_kv = 0 if self.shares_cache else self.kv_heads
        group = batch.groups[cache.group]
        q = torch.empty((tokens, self.q_heads * self.dim), dtype=h.dtype, device=h.device)
        eps = float(self.qk_norm_eps or 0.0)
        table = self.position.tables(batch) if self.position is not None else None
        fused = self.position is None or table is not None
        k_pool, v_pool = (cache.k_pool, cache.v_pool) if own_kv else (None, None)
        heads = self._project_heads
        if (heads is not None and own_kv and table is not None and self.qk_norm_eps is not None
                and heads(h, self.w_qkv, q, k_pool, v_pool, self.q_norm_w, self.k_norm_w, table, group.slot_map,
                          self.q_heads, own_kv, self.dim, cache.page_tokens, eps)):
            return q                       # projection, norm, rotation and page write were one kernel
        qkv = self.runtime.linear(h, self.w_qkv)
        if fused:
            ops.qk_norm_rope_kv(qkv, q, k_pool, v_pool, self.q_norm_w, self.k_norm_w, table, group.slot_map,
                                self.q_heads, own_kv, self.dim, cache.page_tokens, eps)
        else:
            # norm in place, the position encoding as its own step, then the page write
            ops.qk_norm_rope_kv(qkv, q, None, None, self.q_norm_w, self.k_norm_w, None, None,
                                self.q_heads, own_kv, self.dim, cache.page_tokens, eps)
            k_rows = qkv[:, self.q_heads * self.dim:(self.q_heads + own_kv) * self.dim]
            self.position.apply(q.view(tokens, self.q_heads, self.dim),
                                k_rows.unflatten(1, (own_kv, self.dim)) if own_kv else None, batch.positions)
            if own_kv:
                ops.qk_norm_rope_kv(qkv, None, k_pool, v_pool, None, None, None, group.slot_map,
                                    self.q_heads, own_kv, self.dim, cache.page_tokens, eps)
        return q

    def attend(self, q, cache, batch, group, out) -> None:
        self._attend(q, cache, out, group.block_table, batch, self.q_heads, self.kv_heads, self.dim,
                     cache.page_tokens, self.scale, self.window or 0)


def attention_spec(hidden, q_heads, kv_heads, head_dim, qk_norm_eps, theta, names: dict[str, str], window=None,
                   shares_cache=False) -> PartSpec:
    """`names`: the checkpoint's tensor names for q, k, v, o, q_norm, k_norm, relative to the layer's prefix."""
    position = PartSpec("rotary_half", {"dim": head_dim, "theta": theta}) if theta is not None else None
    return PartSpec("attention", {
        "hidden": hidden, "q_heads": q_heads, "kv_heads": kv_heads, "head_dim": head_dim,
        "qk_norm_eps": qk_norm_eps, "position": position, "window": window, "shares_cache": shares_cache, **names,
    })
