"""A plain, slow Vopozen in float64 torch on the CPU: the oracle of the Vopozen tests.

One function per mechanism, written from the design's equations and sharing nothing with the
package: every sequence is taken alone and whole, token by token where the design is a recurrence,
with no cache, no pages and no batching. `forward` returns the logits of every position and the
residual stream after every layer.

Notation: n tokens, W the model width, H query heads, G key/value heads, d the query/key size of a
head, e its value size, r the rotated channels, c the latent size.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def exact(t: torch.Tensor) -> torch.Tensor:
    return t


def through_bfloat16(t: torch.Tensor) -> torch.Tensor:
    """What a tensor becomes when it is stored in bfloat16 (inputs and outputs of matrix products in a
    bfloat16 run); the difference to the exact run says how far such rounding can move a row of logits."""
    return t.to(torch.bfloat16).to(F)


def rms_norm(x: torch.Tensor, weight, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* weight) over the last axis."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


# ----------------------------------------------------------------------------- rotation and masks
def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, heads, d]; the first `dims` channels of every head turn, channel 2i together with channel 2i + 1:
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i / dims). The rest passes."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F) * (base ** (-2.0 * i / dims))
        cos, sin = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * cos - v * sin
        out[:, :, 2 * i + 1] = v * cos + u * sin
    return out


def visible(n: int, kind: str, size: int) -> torch.Tensor:
    """mask[i, j]: whether position i sees position j. "chunk": j <= i in the same chunk of `size` positions counted
    from 0; "window": 0 <= i - j < size."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    if kind == "chunk":
        return (j <= i) & (i // size == j // size)
    return (j <= i) & (i - j < size)


def softmax_attention(q, k, v, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """q [n, H, d], k [n, H, d], v [n, H, e] (already one key/value head per query head) -> [n, H, e]."""
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    scores = scores.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hij,jhe->ihe", torch.softmax(scores, dim=-1), v)


# ----------------------------------------------------------------------------- mixers
def attention_mixer(h, t: dict, m: dict, eps: float, stored=exact) -> torch.Tensor:
    """Grouped-query attention whose values are the key projections themselves (before norm and rotation), a norm per
    q and k head with one weight shared by the heads, neighbouring-pair rotation of the first rot.dims channels, a
    chunked mask."""
    n, H, G, d = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    positions = torch.arange(n)
    q = stored(h @ t["mix.q"].T).view(n, H, d)
    k_raw = stored(h @ t["mix.k"].T).view(n, G, d)
    v = k_raw
    q = rms_norm(q, t["mix.q.norm"], eps)
    k = rms_norm(k_raw, t["mix.k.norm"], eps)
    q = stored(rotate_neighbours(q, positions, m["rot"]["dims"], m["rot"]["base"]))
    k = stored(rotate_neighbours(k, positions, m["rot"]["dims"], m["rot"]["base"]))
    per = H // G
    k, v = k.repeat_interleave(per, dim=1), stored(v).repeat_interleave(per, dim=1)
    out = softmax_attention(q, k, v, m["scale"], visible(n, "chunk", m["mask"]["size"]))
    return stored(stored(out.reshape(n, H * d)) @ t["mix.o"].T)


def latent_rows(h, t: dict, m: dict, eps: float, stored=exact):
    """What a layer with a W_dkv leaves for itself and for the layers that read it: the normed latent [n, c] and the
    rotated key part [n, r]."""
    n, c, r = h.shape[0], m["kv_rank"], m["rot_dim"]
    down = h @ t["mix.dkv"].T
    latent = rms_norm(down[:, :c], t["mix.dkv.norm"], eps)
    k_rot = rotate_neighbours(down[:, None, c:], torch.arange(n), r, m["rot"]["base"])[:, 0]
    return stored(latent), stored(k_rot)


def latent_mixer(h, t: dict, m: dict, eps: float, stored=exact, rows=None):
    """Attention over a latent, written unfolded: every head's keys and values are made from the latent. `rows`: the
    (latent, rotated key part) of the layer this one reads, or None to make its own. Returns (output, rows)."""
    n, H, d, r, e, c = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    if rows is None:
        rows = latent_rows(h, t, m, eps, stored)
    latent, k_rot = rows
    q = (h @ t["mix.q"].T).view(n, H, d + r)
    q_plain, q_rot = q[:, :, :d], rotate_neighbours(q[:, :, d:], torch.arange(n), r, m["rot"]["base"])
    k_plain = (latent @ t["mix.uk"].T).view(n, H, d)
    values = (latent @ t["mix.uv"].T).view(n, H, e)
    q_all = stored(torch.cat((q_plain, q_rot), dim=-1))
    k_all = torch.cat((k_plain, k_rot[:, None, :].expand(n, H, r)), dim=-1)
    out = softmax_attention(q_all, k_all, values, m["scale"], visible(n, "window", m["mask"]["size"]))
    return stored(stored(out.reshape(n, H * e)) @ t["mix.o"].T), rows


def wkv_scan(r, k, v, w, u) -> torch.Tensor:
    """r, k, v, w [n, H, d], u [H, d]: per head o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T,
    S = 0 before the first token."""
    n, H, d = r.shape
    S = torch.zeros((H, d, d), dtype=F)
    out = torch.zeros((n, H, d), dtype=F)
    for t in range(n):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t][:, :, None] * S + kv
    return out


def wkv_mixer(h, t: dict, m: dict, eps: float, stored=exact) -> torch.Tensor:
    """Time mixing with a decay per key channel that depends on the token."""
    n, H, d = h.shape[0], m["heads"], m["dim"]
    before = torch.cat((torch.zeros_like(h[:1]), h[:-1]), dim=0)
    mixed = {s: stored(h + (before - h) * t["mix.mu." + s]) for s in "rkvgw"}
    r = stored(mixed["r"] @ t["mix.r"].T).view(n, H, d)
    k = stored(mixed["k"] @ t["mix.k"].T).view(n, H, d)
    v = stored(mixed["v"] @ t["mix.v"].T).view(n, H, d)
    gate = silu(stored(mixed["g"] @ t["mix.g"].T))
    w = torch.exp(-torch.exp(torch.tanh(mixed["w"] @ t["mix.w1"].T) @ t["mix.w2"].T + t["mix.w0"])).view(n, H, d)
    o = wkv_scan(r, k, v, w, t["mix.u"])
    o = rms_norm(o, None, eps).reshape(n, H * d) * t["mix.norm"] * gate
    return stored(stored(o) @ t["mix.o"].T)


# ----------------------------------------------------------------------------- feed-forwards
def dense_feed_forward(h, t: dict, stored=exact) -> torch.Tensor:
    return stored(stored(silu(h @ t["gate"].T) * (h @ t["up"].T)) @ t["down"].T)


def plain_expert(h, up, down, stored=exact) -> torch.Tensor:
    return stored(stored(torch.relu(h @ up.T) ** 2) @ down.T)


def route(h, t: dict, router: dict):
    """(chosen experts [n, top], their weights [n, top])."""
    n, E, top = h.shape[0], router["experts"], router["top"]
    s = torch.sigmoid(h @ t["router"].T)
    choice = s + t["correction"]
    groups = router.get("groups")
    if groups:
        size = E // groups["count"]
        by_group = choice.view(n, groups["count"], size)
        group_score = by_group.topk(min(2, size), dim=-1).values.sum(dim=-1)
        kept = group_score.topk(groups["keep"], dim=-1).indices
        open_ = torch.zeros((n, groups["count"]), dtype=torch.bool)
        open_.scatter_(1, kept, True)
        choice = choice.masked_fill(~open_[:, :, None].expand(n, groups["count"], size).reshape(n, E), float("-inf"))
    chosen = choice.topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"]


def routed_feed_forward(h, t: dict, mlp: dict, stored=exact) -> torch.Tensor:
    chosen, weights = route(h, t, mlp["router"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, w in zip(chosen[i].tolist(), weights[i].tolist()):
            out[i] += w * plain_expert(h[i: i + 1], t[f"e{e}.up"], t[f"e{e}.down"], stored)[0]
    if mlp.get("shared"):
        out = out + plain_expert(h, t["shared.up"], t["shared.down"], stored)
    return stored(out)


# ----------------------------------------------------------------------------- the model
def forward(config: dict, tensors: dict, tokens: list[int], stored=exact):
    """(logits [n, vocab], the stream after every layer [layers, n, W]) of one whole sequence."""
    eps, m_res = config["norm"]["eps"], config["residual_mult"]
    x = tensors["embed"].to(F)[torch.tensor(tokens)]
    streams, latents = [], {}
    for index, layer in enumerate(config["layers"]):
        t, m = sub(tensors, f"l{index}."), layer["mixer"]
        h = stored(x)
        if layer["type"] == "attention":
            mixed = attention_mixer(h, t, m, eps, stored)
        elif layer["type"] == "latent_attention":
            source = m.get("kv_from")
            mixed, latents[index] = latent_mixer(h, t, m, eps, stored, None if source is None else latents[source])
        else:
            mixed = wkv_mixer(h, t, m, eps, stored)
        x = x + m_res * rms_norm(mixed, t["norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = stored(x)
            ff = sub(tensors, f"l{index}.mlp.")
            out = dense_feed_forward(h, ff, stored) if mlp["kind"] == "dense" else routed_feed_forward(h, ff, mlp, stored)
            x = x + m_res * rms_norm(out, t["norm2"], eps)
        streams.append(x.clone())
    logits = stored(rms_norm(x, tensors["final.norm"].to(F), eps)) @ tensors["head"].to(F).T
    return logits, torch.stack(streams)
