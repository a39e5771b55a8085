"""Typed configuration of Kirenex, read from its own config.json keys.

Kirenex is a decoder whose layers are listed one by one. A learned vector per position is added to the
token embedding. Every layer norms AFTER the sum: x <- norm1(alpha x + mixer(x)), then, where the layer has
a feed-forward, x <- norm2(alpha x + ff(x)), with alpha = `postln_alpha` and RMS norms. Two kinds of layers:

`latent_attention`: attention over a latent of `kv_rank` channels per token plus one rotated key part of
`rot_dim` channels shared by the heads (`heads`, `dim` unrotated and `rot_dim` rotated query/key channels per
head, values of `vdim`, `scale`, `rot` = {base, dims}, neighbouring channels rotate together), full causal
softmax, a sigmoid gate per channel. With `kv_from`: j the layer makes no latent of its own and reads layer j's.

`parallel`: two mixers side by side, averaged after an RMS norm of each. `left` is grouped-query attention
(`heads`, `kv_heads`, `dim`, `vdim`, `scale`) with a norm per head on q and k, a rotation of the first
`rot.dims` channels (halves rotate together; `rot.scaling` = {factor, low, high, original} rescales the
frequencies by wavelength) and a sliding window `mask.size` that keeps the first `mask.keep_first` tokens
visible. `right` is a gated delta rule (`heads`, `kv_heads`, `dim`, `vdim`, `conv` taps).

The feed-forward (`mlp`) is `{"kind": "dense", "ff": N}` (down(gelu_tanh(gate x) * up x)) or null. Other keys:
`vocab`, `width`, `max_positions`, `norm.eps`. Nothing else is read, and nothing that these keys give stands
anywhere in code.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field


def _positive_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value > 0


def _need_ints(where: str, table: dict, keys) -> None:
    for k in keys:
        if not _positive_int(table.get(k)):
            raise ValueError(f"{where}.{k} must be a positive integer, got {table.get(k)!r}")


def _check_rot(where: str, rot, most: int) -> None:
    rot = rot or {}
    if not _positive_int(rot.get("dims")) or rot["dims"] % 2 or rot["dims"] > most or not float(rot.get("base", 0)) > 0:
        raise ValueError(f"{where}: rot needs an even dims <= {most} and a positive base, got {rot!r}")
    scaling = rot.get("scaling")
    if scaling:
        missing = [k for k in ("factor", "low", "high", "original") if k not in scaling]
        if missing:
            raise ValueError(f"{where}: rot.scaling lacks {missing}")
        if not (float(scaling["factor"]) > 0 and float(scaling["high"]) > float(scaling["low"]) >= 0 and float(scaling["original"]) > 0):
            raise ValueError(f"{where}: rot.scaling needs factor > 0, high > low >= 0, original > 0, got {scaling!r}")


@dataclass(frozen=True)
class KirenexConfig:
    vocab: int
    width: int
    layers: tuple            # of dicts {"type", "mixer", "mlp"}, as config.json lists them
    max_positions: int
    postln_alpha: float = 1.0
    norm_eps: float = 1e-6
    eos_token_id: int | None = field(default=None, compare=False)

    architecture = "Kirenex"
    model_type = "kirenex"

    def __post_init__(self):
        _need_ints("config", {"vocab": self.vocab, "width": self.width, "max_positions": self.max_positions},
                   ("vocab", "width", "max_positions"))
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if not self.postln_alpha > 0:
            raise ValueError("postln_alpha must be positive")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for index, layer in enumerate(self.layers):
            where, mixer = f"layer {index}", layer.get("mixer") or {}
            if layer.get("type") == "latent_attention":
                _need_ints(where + ": mixer", mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
                _check_rot(where, mixer.get("rot"), mixer["rot_dim"])
                if mixer["rot"]["dims"] != mixer["rot_dim"]:
                    raise ValueError(f"{where}: the rotated key part is rotated whole: rot.dims must equal rot_dim")
                if not float(mixer.get("scale", 0)) > 0:
                    raise ValueError(f"{where}: mixer.scale must be positive")
                source = mixer.get("kv_from")
                if source is not None:
                    if not isinstance(source, int) or not 0 <= source < index:
                        raise ValueError(f"{where}: kv_from must name an earlier layer, got {source!r}")
                    other = self.layers[source]
                    if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ValueError(f"{where}: kv_from must name a latent_attention layer that makes its own latent")
                    same = ("kv_rank", "rot_dim", "rot")
                    if any(other["mixer"].get(k) != mixer.get(k) for k in same):
                        raise ValueError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {source}")
            elif layer.get("type") == "parallel":
                left, right = mixer.get("left") or {}, mixer.get("right") or {}
                _need_ints(where + ": mixer.left", left, ("heads", "kv_heads", "dim", "vdim"))
                _need_ints(where + ": mixer.right", right, ("heads", "kv_heads", "dim", "vdim", "conv"))
                for side, table in (("left", left), ("right", right)):
                    if table["heads"] % table["kv_heads"]:
                        raise ValueError(f"{where}: {side}.heads ({table['heads']}) must be a multiple of kv_heads ({table['kv_heads']})")
                _check_rot(where + ": left", left.get("rot"), left["dim"])
                if not float(left.get("scale", 0)) > 0:
                    raise ValueError(f"{where}: mixer.left.scale must be positive")
                mask = left.get("mask") or {}
                if not _positive_int(mask.get("size")):
                    raise ValueError(f"{where}: mixer.left.mask.size must be a positive integer")
                keep = mask.get("keep_first", 0)
                if not isinstance(keep, int) or isinstance(keep, bool) or keep < 0:
                    raise ValueError(f"{where}: mixer.left.mask.keep_first must be a non-negative integer")
            else:
                raise ValueError(f"{where}: unknown type {layer.get('type')!r}; known: ['latent_attention', 'parallel']")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ValueError(f"{where}: unknown mlp kind {mlp.get('kind')!r}; known: ['dense']")
                if not _positive_int(mlp.get("ff")):
                    raise ValueError(f"{where}: mlp.ff must be a positive integer")

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "KirenexConfig":
        missing = [k for k in ("vocab", "width", "layers", "max_positions") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        eos = raw.get("eos_token_id")
        return cls(
            vocab=raw["vocab"], width=raw["width"],
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            max_positions=raw["max_positions"],
            postln_alpha=float(raw.get("postln_alpha", 1.0)),
            norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
            eos_token_id=eos[0] if isinstance(eos, list) else eos,
        )

    def to_hf_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        return {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "max_positions": self.max_positions,
            "norm": {"eps": self.norm_eps},
            "postln_alpha": self.postln_alpha,
            "vocab": self.vocab,
            "width": self.width,
        }


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None, kv_from=None, ff=None) -> dict:
    """One `latent_attention` entry of `layers`."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel_layer(heads, kv_heads, dim, vdim, window, keep_first=0, rot_dims=None, base=10000.0, scaling=None, scale=None,
                   delta_heads=2, delta_kv_heads=None, delta_dim=16, delta_vdim=16, taps=4, ff=None) -> dict:
    """One `parallel` entry of `layers`: windowed attention on the left, a gated delta rule on the right."""
    rot = {"base": base, "dims": rot_dims or dim}
    if scaling:
        rot["scaling"] = dict(scaling)
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot,
            "mask": {"size": window, "keep_first": keep_first}, "scale": scale if scale is not None else dim ** -0.5}
    right = {"heads": delta_heads, "kv_heads": delta_kv_heads or delta_heads, "dim": delta_dim, "vdim": delta_vdim, "conv": taps}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# Named shapes for the command line and the benchmark (inputs, like a parsed config.json).
KIRENEX_PRESETS: dict[str, dict] = {
    "kirenex-tiny": dict(
        vocab=352, width=112, max_positions=512, postln_alpha=1.5, norm_eps=1e-5,
        layers=(latent_layer(3, 24, 8, 40, 48, base=20000.0, ff=144),
                parallel_layer(4, 2, 32, 48, 40, keep_first=6, rot_dims=16, scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64},
                               delta_heads=4, delta_kv_heads=2, delta_dim=24, delta_vdim=40, taps=4, ff=208),
                latent_layer(2, 16, 8, 24, 48, base=20000.0, kv_from=0),
                parallel_layer(2, 1, 48, 32, 24, keep_first=0, delta_heads=2, delta_dim=32, delta_vdim=16, taps=2, ff=96))),
}
