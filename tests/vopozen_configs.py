"""Small Vopozen configurations for the tests: sizes differ from layer to layer, and values that could hide a
fault by being equal (head counts, rotated channels and head size, the windows of a latent and of the layer that
reads it, kept groups and all groups) or by being 1 (the multiplier, a window, a chunk, the chosen experts, a
decay rank) are mixed on purpose."""

from __future__ import annotations


def moe(experts, top, ff, scale, groups=None, keep=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def attention(heads, kv_heads, dim, chunk, rot_dims, base, scale, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk},
                      "rot": {"base": base, "dims": rot_dims}, "scale": scale}}


def latent(heads, dim, rot_dim, vdim, rank, window, base, scale, kv_from=None, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": window},
             "rot": {"base": base, "dims": rot_dim}, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def wkv(heads, dim, rank, mlp=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp}


def config(vocab, width, layers, mult, eps=1e-5):
    return {"architecture": "Vopozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


CONFIGS = {
    # head sizes that are no multiple of 16 or of 4 (the 32-bit attention kernel on padded rows in both precisions for
    # the chunks, padded tensor-core rows for the latent); a latent that a later layer reads through a WIDER window than
    # its own; routed experts in groups of three of which two are kept, and without groups; a layer without a feed-forward
    "odd_sizes": config(211, 72, [
        wkv(3, 12, 5, dense(96)),
        latent(3, 12, 6, 20, 36, 9, 5000.0, 0.3, mlp=moe(6, 2, 40, 1.5, groups=2, keep=1, shared=56)),
        attention(4, 2, 12, 24, 8, 300.0, 0.35, mlp=dense(80)),
        latent(2, 8, 6, 10, 36, 33, 5000.0, 0.4, kv_from=1),
        wkv(2, 20, 3, moe(5, 1, 24, 0.7)),
        attention(2, 1, 24, 7, 24, 1000.0, 0.2, mlp=moe(9, 4, 16, 2.5, groups=3, keep=2)),
    ], mult=0.6),
    # head sizes that are multiples of 16: the tensor-core kernels in bfloat16; a latent read by the layer right behind
    # it (through a NARROWER window) and by the last one; groups of two experts (a group's score is all of it); eight
    # query heads on one key/value head; two wkv layers of different head sizes
    "wide_heads": config(150, 96, [
        attention(8, 1, 32, 40, 16, 20000.0, 0.2, mlp=moe(8, 3, 48, 2.0, groups=4, keep=2, shared=64)),
        latent(4, 16, 16, 32, 48, 24, 10000.0, 0.25, mlp=dense(64)),
        latent(2, 32, 16, 16, 48, 5, 10000.0, 0.2, kv_from=1, mlp=dense(48)),
        wkv(2, 64, 16, dense(112)),
        attention(6, 2, 64, 64, 32, 10000.0, 0.15, mlp=dense(80)),
        wkv(3, 32, 32, moe(4, 2, 32, 1.0, shared=32)),
        latent(5, 16, 16, 48, 48, 40, 10000.0, 0.3, kv_from=1),
    ], mult=1.0, eps=1e-6),
    # one layer of each kind, one head, a window and a chunk of 1 (a token sees itself only), a decay rank of 1, every
    # expert chosen, twenty query heads on one latent (more than a tile of the decode kernel holds)
    "smallest": config(64, 32, [
        attention(1, 1, 16, 1, 2, 100.0, 1.0),
        wkv(1, 4, 1, moe(2, 2, 8, 3.0)),
        latent(20, 4, 2, 4, 6, 1, 100.0, 0.5, mlp=dense(24)),
    ], mult=2.0),
    # a window and a chunk longer than any request; a whole head rotated; all groups kept
    "one_window": config(97, 48, [
        latent(2, 16, 8, 16, 24, 1000, 10000.0, 0.2, mlp=moe(8, 2, 24, 1.0, groups=4, keep=4)),
        wkv(3, 16, 8),
        attention(3, 3, 16, 1000, 16, 10000.0, 0.25, mlp=dense(40)),
    ], mult=0.3),
}
PAGES = {"odd_sizes": 4, "wide_heads": 16, "smallest": 2, "one_window": 8}
# the scale of the random weights: as large as leaves the plain model itself well conditioned
INIT = {name: dict(std=0.1 if name == "wide_heads" else 0.2, norm_std=0.3) for name in CONFIGS}
