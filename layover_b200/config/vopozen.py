"""Typed configuration of Vopozen, read from its own config.json keys.

Vopozen is a decoder whose layers are listed one by one. Every layer norms a sub-layer's OUTPUT only:
x <- x + m * norm1(mixer(x)), then, where the layer has a feed-forward, x <- x + m * norm2(ff(x)), with
m = `residual_mult` and RMS norms; the sub-layers read the stream itself. Three kinds of layers (`type`):

`attention`: grouped-query attention (`heads`, `kv_heads`, `dim`, `vdim`, `scale`) whose values are the key
projections themselves (no value matrix; `vdim` equals `dim`), an RMS norm per q and k head, a rotation of the
first `rot.dims` channels of a head (neighbouring channels turn together, frequencies `rot.base`^(-2i/dims)) and
a chunked mask: a query sees the earlier keys of its own chunk of `mask.size` positions.

`latent_attention`: attention over a latent of `kv_rank` channels per token plus one rotated key part of
`rot_dim` channels shared by the heads (`heads`, `dim` unrotated and `rot_dim` rotated query/key channels per
head, values of `vdim`, `scale`, `rot` = {base, dims = rot_dim}), over a sliding window of `mask.size` tokens.
With `kv_from`: j the layer makes no latent of its own and reads layer j's.

`wkv`: time mixing with token shift and a decay per token and key channel (`heads`, `dim`). The rank of the decay's
two small matrices is the one size that config.json may leave to the stored tensors (`decay_rank`, else the
rows of `l<i>.mix.w1`).

The feed-forward (`mlp`) is `{"kind": "dense", "ff": N}` (down(silu(gate x) * up x)), `{"kind": "moe", "router":
{experts, top, scale, groups: {count, keep}}, "expert": {ff}, "shared": {ff}}` (a mixture of ungated experts
down(relu(up x)^2), sigmoid scores, a correction added for the choice only, the choice limited to the best
groups of neighbouring experts, the chosen scores normalised and scaled, a shared expert for every token), or
null. Other keys: `vocab`, `width`, `norm.eps`, `residual_mult`. Nothing else is read, and nothing that these
keys give stands anywhere in code.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .kirenex import _check_rot, _need_ints, _positive_int

LAYER_TYPES = ("attention", "latent_attention", "wkv")


def _check_mlp(where: str, mlp) -> None:
    if mlp is None:
        return
    kind = mlp.get("kind")
    if kind == "dense":
        if not _positive_int(mlp.get("ff")):
            raise ValueError(f"{where}: mlp.ff must be a positive integer")
        return
    if kind != "moe":
        raise ValueError(f"{where}: unknown mlp kind {kind!r}; known: ['dense', 'moe']")
    router = mlp.get("router") or {}
    _need_ints(where + ": mlp.router", router, ("experts", "top"))
    _need_ints(where + ": mlp.expert", mlp.get("expert") or {}, ("ff",))
    if router["top"] > router["experts"]:
        raise ValueError(f"{where}: mlp.router.top ({router['top']}) exceeds the experts ({router['experts']})")
    if not float(router.get("scale", 1.0)) > 0:
        raise ValueError(f"{where}: mlp.router.scale must be positive")
    groups = router.get("groups")
    if groups:
        _need_ints(where + ": mlp.router.groups", groups, ("count", "keep"))
        if router["experts"] % groups["count"] or groups["keep"] > groups["count"]:
            raise ValueError(f"{where}: the experts ({router['experts']}) form {groups['count']} equal groups of which "
                             f"{groups['keep']} are kept: the counts do not fit")
        if groups["keep"] * (router["experts"] // groups["count"]) < router["top"]:
            raise ValueError(f"{where}: the kept groups hold fewer experts than a token chooses")
    if mlp.get("shared"):
        _need_ints(where + ": mlp.shared", mlp["shared"], ("ff",))


@dataclass(frozen=True)
class VopozenConfig:
    vocab: int
    width: int
    layers: tuple            # of dicts {"type", "mixer", "mlp"}, as config.json lists them
    residual_mult: float = 1.0
    norm_eps: float = 1e-6
    eos_token_id: int | None = field(default=None, compare=False)

    architecture = "Vopozen"
    model_type = "vopozen"
    reads_shapes = True

    def __post_init__(self):
        _need_ints("config", {"vocab": self.vocab, "width": self.width}, ("vocab", "width"))
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if not self.residual_mult > 0:
            raise ValueError("residual_mult must be positive")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for index, layer in enumerate(self.layers):
            where, mixer, kind = f"layer {index}", layer.get("mixer") or {}, layer.get("type")
            if kind == "attention":
                _need_ints(where + ": mixer", mixer, ("heads", "kv_heads", "dim"))
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ValueError(f"{where}: heads ({mixer['heads']}) must be a multiple of kv_heads ({mixer['kv_heads']})")
                if mixer.get("vdim", mixer["dim"]) != mixer["dim"]:
                    raise ValueError(f"{where}: the values are the keys, so vdim must equal dim")
                _check_rot(where, mixer.get("rot"), mixer["dim"])
            elif kind == "latent_attention":
                _need_ints(where + ": mixer", mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
                _check_rot(where, mixer.get("rot"), mixer["rot_dim"])
                if mixer["rot"]["dims"] != mixer["rot_dim"]:
                    raise ValueError(f"{where}: the rotated key part is rotated whole: rot.dims must equal rot_dim")
                source = mixer.get("kv_from")
                if source is not None:
                    if not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < index:
                        raise ValueError(f"{where}: kv_from must name an earlier layer, got {source!r}")
                    other = self.layers[source]
                    if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ValueError(f"{where}: kv_from must name a latent_attention layer that makes its own latent")
                    if any(other["mixer"].get(k) != mixer.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        raise ValueError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {source}")
            elif kind == "wkv":
                _need_ints(where + ": mixer", mixer, ("heads", "dim", "decay_rank"))
            else:
                raise ValueError(f"{where}: unknown type {kind!r}; known: {list(LAYER_TYPES)}")
            if kind != "wkv":
                if not float(mixer.get("scale", 0)) > 0:
                    raise ValueError(f"{where}: mixer.scale must be positive")
                if not _positive_int((mixer.get("mask") or {}).get("size")):
                    raise ValueError(f"{where}: mixer.mask.size must be a positive integer")
            _check_mlp(where, layer.get("mlp"))

    @classmethod
    def from_hf_dict(cls, raw: dict, shapes: dict | None = None) -> "VopozenConfig":
        """`shapes` (tensor name -> shape of the stored tensors) fills in what config.json leaves to them: the rank of a
        wkv layer's decay matrices."""
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        layers = tuple(copy.deepcopy(layer) for layer in raw["layers"])
        for index, layer in enumerate(layers):
            if layer.get("type") == "wkv" and isinstance(layer.get("mixer"), dict) and "decay_rank" not in layer["mixer"]:
                shape = (shapes or {}).get(f"l{index}.mix.w1")
                if shape is None:
                    raise ValueError(f"layer {index}: mixer.decay_rank is neither in config.json nor given by a stored l{index}.mix.w1")
                layer["mixer"]["decay_rank"] = int(shape[0])
        eos = raw.get("eos_token_id")
        return cls(
            vocab=raw["vocab"], width=raw["width"], layers=layers,
            residual_mult=float(raw.get("residual_mult", 1.0)),
            norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
            eos_token_id=eos[0] if isinstance(eos, list) else eos,
        )

    def to_hf_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        return {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }


def _mlp(ff=None, experts=None, top=1, expert_ff=None, shared_ff=None, groups=None, keep=None, route_scale=1.0):
    if experts:
        router = {"experts": experts, "top": top, "scale": route_scale}
        if groups:
            router["groups"] = {"count": groups, "keep": keep or groups}
        mlp = {"kind": "moe", "router": router, "expert": {"ff": expert_ff}}
        if shared_ff:
            mlp["shared"] = {"ff": shared_ff}
        return mlp
    return {"kind": "dense", "ff": ff} if ff else None


def chunked_layer(heads, kv_heads, dim, chunk, rot_dims=None, base=10000.0, scale=None, **mlp) -> dict:
    """One `attention` entry of `layers`."""
    return {"type": "attention", "mlp": _mlp(**mlp),
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk},
                      "rot": {"base": base, "dims": rot_dims or dim}, "scale": scale if scale is not None else dim ** -0.5}}


def windowed_latent_layer(heads, dim, rot_dim, vdim, kv_rank, window, base=10000.0, scale=None, kv_from=None, **mlp) -> dict:
    """One `latent_attention` entry of `layers`."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
             "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": _mlp(**mlp)}


def wkv_layer(heads, dim, decay_rank, **mlp) -> dict:
    """One `wkv` entry of `layers`."""
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}, "mlp": _mlp(**mlp)}


# Named shapes for the command line and the benchmark (inputs, like a parsed config.json).
VOPOZEN_PRESETS: dict[str, dict] = {
    "vopozen-tiny": dict(
        vocab=320, width=96, norm_eps=1e-5, residual_mult=0.5,
        layers=(wkv_layer(3, 16, 8, ff=160),
                chunked_layer(4, 2, 32, 24, rot_dims=16, base=50000.0,
                              experts=8, top=2, expert_ff=48, shared_ff=64, groups=4, keep=2, route_scale=1.5),
                windowed_latent_layer(3, 24, 8, 40, 48, 20, base=20000.0, ff=128),
                windowed_latent_layer(2, 16, 8, 24, 48, 36, base=20000.0, kv_from=2,
                                      experts=6, top=3, expert_ff=32, route_scale=2.5),
                wkv_layer(2, 24, 12))),
}
