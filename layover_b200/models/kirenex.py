"""Kirenex as a list of layers: a learned vector per position joins the token embedding; every layer norms
AFTER the sum (x <- norm(alpha x + sub-layer(x)), the sub-layers read the stream itself) around one of two
mixers and a gelu-gated feed-forward or none. The mixers: attention over a latent (one small normed vector and
one rotated key part per token in the cache, a sigmoid gate per channel; a layer may read an earlier layer's
latent instead of making its own), or two mixers side by side whose normed outputs are averaged: grouped-query
attention with a norm per head, a partial rotation with banded frequencies and a window that keeps the first
tokens, beside a gated delta rule behind short convolutions. The residual stream is 32-bit in either precision.
Tensor names are the checkpoint's own: `embed`, `pos`, `l<i>.norm1 / norm2`, `l<i>.mix.*` (`left.*`, `right.*`
under a side-by-side mixer), `l<i>.mlp.{gate,up,down}`, `final.norm`, `head`."""

from __future__ import annotations

from ..config.base import register_architecture
from ..config.kirenex import KirenexConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry


def _latent(cfg: KirenexConfig, m: dict) -> PartSpec:
    return PartSpec("latent_attention", {
        "hidden": cfg.width, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
        "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "norm_eps": cfg.norm_eps,
        "shares_cache": m.get("kv_from") is not None,
        "position": PartSpec("rotary_pairs", {"dim": m["rot_dim"], "theta": float(m["rot"]["base"]), "rotated": int(m["rot"]["dims"])}),
        "q": "mix.q", "down": "mix.dkv", "down_norm": "mix.dkv.norm", "up_k": "mix.uk", "up_v": "mix.uv", "gate": "mix.g", "o": "mix.o"})


def _side_by_side(cfg: KirenexConfig, m: dict) -> PartSpec:
    left, right = m["left"], m["right"]
    rot = left["rot"]
    attention = PartSpec("attention", {
        "hidden": cfg.width, "q_heads": left["heads"], "kv_heads": left["kv_heads"], "head_dim": left["dim"],
        "v_head_dim": left["vdim"], "scale": float(left["scale"]), "window": int(left["mask"]["size"]),
        "keep_first": int(left["mask"].get("keep_first", 0)), "qk_norm_eps": cfg.norm_eps, "exact_weights": True,
        "position": PartSpec("rotary_half", {"dim": left["dim"], "theta": float(rot["base"]), "rotated": int(rot["dims"]),
                                             "band_scaling": rot.get("scaling")}),
        "q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"})
    delta = PartSpec("gated_delta_rule", {
        "hidden": cfg.width, "heads": right["heads"], "kv_heads": right["kv_heads"], "head_dim": right["dim"],
        "v_head_dim": right["vdim"], "taps": right["conv"], "norm_eps": cfg.norm_eps,
        "q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a": "a",
        "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "o": "o"})
    return PartSpec("side_by_side", {"hidden": cfg.width, "eps": cfg.norm_eps,
                                     "mixers": [(attention, "mix.left.", "mix.left.out"), (delta, "mix.right.", "mix.right.out")]})


def kirenex_spec(cfg: KirenexConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": cfg.width, "eps": cfg.norm_eps, "weight": weight})

    layers, schedule, ignorable = [], [], set()
    for index, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        mixer = _latent(cfg, m) if layer["type"] == "latent_attention" else _side_by_side(cfg, m)
        mlp = layer.get("mlp")
        block = PartSpec("post_norm", {
            "alpha": cfg.postln_alpha, "mixer": mixer, "mixer_norm": norm("norm1"),
            "feed_forward": PartSpec("gated_mlp", {"hidden": cfg.width, "inter": mlp["ff"], "activation": "gelu_tanh",
                                                   "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}) if mlp else None,
            "ff_norm": norm("norm2") if mlp else None})
        layers.append(LayerSpec(block, f"l{index}."))
        if not mlp:
            ignorable.add(f"l{index}.norm2")       # may be stored for every layer; unused where nothing follows the mixer
        # one schedule entry per layer, so a layer's index is also its entry's
        schedule.append(ScheduleEntry(index, reads_cache_of=m.get("kv_from") if layer["type"] == "latent_attention" else None))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_position=cfg.max_positions,
        embedding="embed",
        position_table="pos",
        final_norm=norm("final.norm"),
        head="head",
        layers=layers,
        schedule=schedule,
        residual_dtype="float32",
        ignorable_tensors=frozenset(ignorable),
    )


register_architecture(KirenexConfig.architecture, KirenexConfig.model_type, KirenexConfig, kirenex_spec)
