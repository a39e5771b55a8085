"""Vopozen as a list of layers: every layer norms a sub-layer's OUTPUT only and adds it times a constant
(x <- x + m * norm(sub-layer(x)); the sub-layers read the stream itself) around one of three mixers and a
feed-forward or none. The mixers: grouped-query attention whose values are its key projections, with a norm per
head, a partial rotation of neighbouring channels and a chunked mask; attention over a latent within a sliding
window (a layer may read an earlier layer's latent instead of making its own); time mixing with token shift and a
decay per token and key channel. The feed-forward is a silu-gated one or a mixture of ungated squared-relu experts
whose choice is corrected, limited to groups and renormalised, with a shared expert. The residual stream is 32-bit
in either precision. Tensor names are the checkpoint's own: `embed`, `l<i>.norm1 / norm2`, `l<i>.mix.*`,
`l<i>.mlp.*`, `final.norm`, `head`."""

from __future__ import annotations

from ..config.base import register_architecture
from ..config.vopozen import VopozenConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

# the rotation's angles are 32-bit products of position and frequency; the cache bounds a request's length
UNBOUNDED_POSITIONS = 1 << 30


def _attention(cfg: VopozenConfig, m: dict) -> PartSpec:
    rot = m["rot"]
    return PartSpec("attention", {
        "hidden": cfg.width, "q_heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "values": "keys",
        "scale": float(m["scale"]), "chunk": int(m["mask"]["size"]), "qk_norm_eps": cfg.norm_eps,
        "position": PartSpec("rotary_pairs", {"dim": m["dim"], "theta": float(rot["base"]), "rotated": int(rot["dims"])}),
        "q": "mix.q", "k": "mix.k", "o": "mix.o", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm"})


def _latent(cfg: VopozenConfig, m: dict, cache_window: int) -> PartSpec:
    return PartSpec("latent_attention", {
        "hidden": cfg.width, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
        "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "norm_eps": cfg.norm_eps,
        "window": int(m["mask"]["size"]), "cache_window": cache_window, "shares_cache": m.get("kv_from") is not None,
        "position": PartSpec("rotary_pairs", {"dim": m["rot_dim"], "theta": float(m["rot"]["base"]), "rotated": int(m["rot"]["dims"])}),
        "q": "mix.q", "down": "mix.dkv", "down_norm": "mix.dkv.norm", "up_k": "mix.uk", "up_v": "mix.uv", "gate": None, "o": "mix.o"})


def _wkv(cfg: VopozenConfig, m: dict) -> PartSpec:
    return PartSpec("wkv", {
        "hidden": cfg.width, "heads": m["heads"], "head_dim": m["dim"], "decay_rank": m["decay_rank"], "norm_eps": cfg.norm_eps,
        "mu_r": "mix.mu.r", "mu_k": "mix.mu.k", "mu_v": "mix.mu.v", "mu_g": "mix.mu.g", "mu_w": "mix.mu.w",
        "r": "mix.r", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "w1": "mix.w1", "w2": "mix.w2", "w0": "mix.w0",
        "u": "mix.u", "norm": "mix.norm", "o": "mix.o"})


def _feed_forward(cfg: VopozenConfig, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"hidden": cfg.width, "inter": mlp["ff"], "activation": "silu",
                                      "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
    router, shared = mlp["router"], mlp.get("shared")
    groups = router.get("groups") or {}
    return PartSpec("routed_experts", {
        "hidden": cfg.width, "experts": router["experts"], "top": router["top"], "inter": mlp["expert"]["ff"],
        "gated": False, "activation": "relu2", "score": "sigmoid", "weight_on": "output", "renormalize": True,
        "route_scale": float(router.get("scale", 1.0)), "groups": groups.get("count"), "keep_groups": groups.get("keep"),
        "correction": "mlp.correction", "router": "mlp.router", "expert_up": "mlp.e{}.up", "expert_down": "mlp.e{}.down",
        "shared": PartSpec("mlp", {"hidden": cfg.width, "inter": shared["ff"], "activation": "relu2",
                                   "up": "mlp.shared.up", "down": "mlp.shared.down"}) if shared else None})


def vopozen_spec(cfg: VopozenConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": cfg.width, "eps": cfg.norm_eps, "weight": weight})

    # a latent's rows are kept for the widest window among the layer that makes them and the layers that read them
    kept = {}
    for index, layer in enumerate(cfg.layers):
        if layer["type"] == "latent_attention":
            owner = layer["mixer"].get("kv_from", index)
            owner = index if owner is None else owner
            kept[owner] = max(kept.get(owner, 0), int(layer["mixer"]["mask"]["size"]))
    layers, schedule, ignorable = [], [], set()
    for index, layer in enumerate(cfg.layers):
        m, reads = layer["mixer"], None
        if layer["type"] == "attention":
            mixer = _attention(cfg, m)
        elif layer["type"] == "latent_attention":
            reads = m.get("kv_from")
            mixer = _latent(cfg, m, kept[index if reads is None else reads])
        else:
            mixer = _wkv(cfg, m)
        mlp = layer.get("mlp")
        block = PartSpec("output_norm", {"mult": cfg.residual_mult, "mixer": mixer, "mixer_norm": norm("norm1"),
                                         "feed_forward": _feed_forward(cfg, mlp), "ff_norm": norm("norm2") if mlp else None})
        layers.append(LayerSpec(block, f"l{index}."))
        if not mlp:
            ignorable.add(f"l{index}.norm2")       # may be stored for every layer; unused where nothing follows the mixer
        schedule.append(ScheduleEntry(index, reads_cache_of=reads))      # one entry per layer: a layer's index is its entry's
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_position=UNBOUNDED_POSITIONS,
        embedding="embed",
        final_norm=norm("final.norm"),
        head="head",
        layers=layers,
        schedule=schedule,
        residual_dtype="float32",
        ignorable_tensors=frozenset(ignorable),
    )


register_architecture(VopozenConfig.architecture, VopozenConfig.model_type, VopozenConfig, vopozen_spec)
