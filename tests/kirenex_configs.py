"""Small Kirenex configurations for the tests: sizes differ from layer to layer, and values that could hide a
fault by being equal (key and value sizes, query and key/value head counts, rotated channels and head size,
the layer a latent is read from and the layer before) or by being 1 or 0 (alpha, taps, kept tokens) are mixed
on purpose."""

from __future__ import annotations


def latent(heads, dim, rot_dim, vdim, rank, base, scale, kv_from=None, ff=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
             "rot": {"base": base, "dims": rot_dim}, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel(left, right, ff=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def left(heads, kv_heads, dim, vdim, window, keep, rot_dims, base, scale, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mask = {"size": window}
    if keep is not None:
        mask["keep_first"] = keep
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "mask": mask, "scale": scale}


def right(heads, kv_heads, dim, vdim, taps):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}


def config(vocab, width, layers, alpha, eps=1e-5, positions=512):
    return {"architecture": "Kirenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "max_positions": positions, "layers": layers}


CONFIGS = {
    # starts with a latent layer that a later one reads; head sizes that are no multiple of 16 or of 4 (the 32-bit
    # attention kernel on padded rows in both precisions for the window, padded tensor-core rows for the latent);
    # two query/key heads for four value heads in the delta rule; a layer without a feed-forward; frequencies in
    # all three bands of the scaling
    "odd_sizes": config(211, 72, [
        latent(3, 12, 6, 20, 36, 5000.0, 0.3, ff=96),
        parallel(left(4, 2, 12, 20, 24, 5, 8, 300.0, 0.35, scaling=(4.0, 1.0, 4.0, 64)), right(4, 2, 12, 20, 4), ff=80),
        latent(2, 8, 6, 10, 36, 5000.0, 0.4, kv_from=0),
        parallel(left(2, 1, 24, 8, 9, 0, 24, 1000.0, 0.2), right(3, 3, 10, 6, 2)),
    ], alpha=1.5),
    # head sizes that are multiples of 16: the tensor-core attention in bfloat16, keys and values of different
    # sizes on pages of the larger size; more kept tokens than the window is long, kept tokens that end on a page
    # border; the latent is read by the layer right behind it and by the last one
    "wide_heads": config(150, 96, [
        parallel(left(4, 1, 32, 16, 7, 16, 16, 20000.0, 0.2, scaling=(8.0, 1.0, 2.0, 32)), right(2, 1, 32, 48, 3), ff=112),
        latent(4, 16, 16, 32, 48, 10000.0, 0.25, ff=64),
        latent(2, 32, 16, 16, 48, 10000.0, 0.2, kv_from=1, ff=48),
        parallel(left(6, 2, 64, 48, 40, 3, 32, 10000.0, 0.15), right(4, 4, 16, 16, 5), ff=80),
        latent(5, 16, 16, 48, 48, 10000.0, 0.3, kv_from=1),
    ], alpha=1.0, eps=1e-6),
    # one layer of each kind, one head, a window of 1 (a token sees itself and the kept first ones), one tap (no
    # convolution at all), twenty query heads on one latent (more than a tile of the decode kernel holds)
    "smallest": config(64, 32, [
        parallel(left(1, 1, 16, 4, 1, 2, 2, 100.0, 1.0), right(1, 1, 4, 8, 1)),
        latent(20, 4, 2, 4, 6, 100.0, 0.5, ff=24),
    ], alpha=3.0),
    # a window longer than any request and no kept tokens named at all; equal key and value sizes, a whole head rotated
    "one_window": config(97, 48, [
        latent(2, 16, 8, 16, 24, 10000.0, 0.2, ff=72),
        parallel(left(3, 3, 16, 16, 1000, None, 16, 10000.0, 0.25, scaling=(2.0, 1.0, 8.0, 16)), right(2, 2, 16, 16, 4), ff=40),
    ], alpha=0.5),
}
PAGES = {"odd_sizes": 4, "wide_heads": 16, "smallest": 2, "one_window": 8}
# the scale of the random weights: as large as leaves the plain model itself well conditioned (run in 32-bit floats it
# then stays within a quarter of the tests' 32-bit tolerance of its 64-bit self; the five-layer model needs smaller weights for that)
INIT = {name: dict(std=0.1 if name == "wide_heads" else 0.2, norm_std=0.3) for name in CONFIGS}
