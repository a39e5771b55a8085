"""A plain, slow Kirenex in float64 torch on the CPU: the oracle of the Kirenex tests.

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


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ----------------------------------------------------------------------------- rotations
def plain_frequencies(base: float, dims: int) -> torch.Tensor:
    """f_i = base^(-2i/dims), i = 0 .. dims/2 - 1."""
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)


def banded_frequencies(base: float, dims: int, scaling: dict | None) -> torch.Tensor:
    """The frequencies above, rescaled by wavelength l = 2 pi / f: short waves (l < original / high) stay,
    long ones (l > original / low) are divided by `factor`, and between the two a frequency is the blend
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    f = plain_frequencies(base, dims)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i, fi in enumerate(f.tolist()):
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_split_halves(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [n, heads, d]; the first 2 len(freq) channels of every head turn, channel i together with channel
    i + len(freq): (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * f_i."""
    half = freq.shape[0]
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]), dim=-1)


def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [n, heads, d]; the first 2 len(freq) channels of every head turn, channel 2i together with channel
    2i + 1, by the same rule."""
    half = freq.shape[0]
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
    out[..., 0:2 * half:2] = u * cos - v * sin
    out[..., 1:2 * half:2] = v * cos + u * sin
    return out


# ----------------------------------------------------------------------------- softmax attention
def masked_softmax_attention(q, k, v, scale: float, window: int | None = None, keep_first: int = 0) -> torch.Tensor:
    """q [n, H, d], k [n, G, d], v [n, G, e] -> [n, H, e]. Query i sees key j <= i; with a window only where
    i - j < window or j < keep_first."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(n, heads, v.shape[2], dtype=F)
    for i in range(n):
        seen = [j for j in range(i + 1) if window is None or i - j < window or j < keep_first]
        for h in range(heads):
            g = h // group
            s = (k[seen, g] @ q[i, h]) * scale
            w = torch.softmax(s, dim=0)
            out[i, h] = (w[:, None] * v[seen, g]).sum(0)
    return out


def windowed_mixer(h, t: dict, m: dict, eps: float, stored=exact) -> torch.Tensor:
    """Grouped-query attention with a per-head RMS norm of q and k before a half-split rotation of the first
    channels (banded frequencies), a window that keeps the first tokens, values of their own size."""
    heads, kv, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    positions = torch.arange(n)
    freq = banded_frequencies(float(m["rot"]["base"]), int(m["rot"]["dims"]), m["rot"].get("scaling"))
    q = rms_norm(stored(h @ t["q"].T).view(n, heads, d), t["q.norm"], eps)
    k = rms_norm(stored(h @ t["k"].T).view(n, kv, d), t["k.norm"], eps)
    q, k = stored(rotate_split_halves(q, positions, freq)), stored(rotate_split_halves(k, positions, freq))
    v = stored(h @ t["v"].T).view(n, kv, e)
    o = masked_softmax_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0)))
    return stored(stored(o.reshape(n, heads * e)) @ t["o"].T)


def latent_mixer(h, t: dict, m: dict, eps: float, stored=exact, shared=None):
    """Attention over a latent: one small vector c per token (RMS-normed) from which every head's unrotated
    keys and its values are made, and one rotated key part that all heads share. Returns the output and
    (c, rotated key part), which a later layer may use instead of making its own (`shared`)."""
    heads, d, r, e, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    positions = torch.arange(n)
    freq = plain_frequencies(float(m["rot"]["base"]), int(m["rot"]["dims"]))
    q = stored(h @ t["q"].T).view(n, heads, d + r)
    q_plain, q_turn = q[..., :d], stored(rotate_neighbours(q[..., d:], positions, freq))
    if shared is None:
        down = stored(h @ t["dkv"].T)
        c = stored(rms_norm(down[:, :rank], t["dkv.norm"], eps))
        k_turn = stored(rotate_neighbours(down[:, None, rank:], positions, freq))[:, 0]
    else:
        c, k_turn = shared
    k_plain = stored(c @ t["uk"].T).view(n, heads, d)
    v = stored(c @ t["uv"].T).view(n, heads, e)
    k = torch.cat((k_plain, k_turn[:, None, :].expand(n, heads, r)), dim=-1)
    o = masked_softmax_attention(torch.cat((q_plain, q_turn), dim=-1), k, v, float(m["scale"]))
    gate = torch.sigmoid(stored(h @ t["g"].T))
    return stored(stored(o.reshape(n, heads * e) * gate) @ t["o"].T), (c, k_turn)


# ----------------------------------------------------------------------------- gated delta rule
def causal_short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [n, channels], taps [channels, k]: y_t = sum_j taps[:, k - 1 - j] x_(t - j), zeros before the start."""
    n, k = x.shape[0], taps.shape[1]
    padded = torch.cat((torch.zeros(k - 1, x.shape[1], dtype=F), x), dim=0)
    return sum(padded[j:j + n] * taps[:, j] for j in range(k))


def delta_rule_scan(q, k, v, beta, decay) -> torch.Tensor:
    """q, k [n, H, d], v [n, H, e], beta, decay [n, H] -> [n, H, e], token by token with S (d x e) from zero:
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n, heads, d = q.shape
    out = torch.zeros(n, heads, v.shape[2], dtype=F)
    for h in range(heads):
        state = torch.zeros(d, v.shape[2], dtype=F)
        for i in range(n):
            state = decay[i, h] * state
            u = beta[i, h] * (v[i, h] - state.T @ k[i, h])
            state = state + torch.outer(k[i, h], u)
            out[i, h] = state.T @ q[i, h]
    return out


def delta_mixer(h, t: dict, m: dict, eps: float, stored=exact) -> torch.Tensor:
    heads, kv, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = stored(silu(stored(causal_short_convolution(stored(h @ t["q"].T), t["q.conv"])))).view(n, kv, d)
    k = stored(silu(stored(causal_short_convolution(stored(h @ t["k"].T), t["k.conv"])))).view(n, kv, d)
    v = stored(silu(stored(causal_short_convolution(stored(h @ t["v"].T), t["v.conv"])))).view(n, heads, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    group = heads // kv
    q, k = q.repeat_interleave(group, dim=1), k.repeat_interleave(group, dim=1)
    beta = torch.sigmoid(stored(h @ t["b"].T))
    decay = torch.exp(-torch.exp(t["A_log"]) * softplus(stored(h @ t["a"].T) + t["dt_bias"]))
    o = delta_rule_scan(q, k, v, beta, decay)
    o = rms_norm(o, t["norm"], eps) * silu(stored(h @ t["g"].T)).view(n, heads, e)
    return stored(stored(o.reshape(n, heads * e)) @ t["o"].T)


def side_by_side_mixer(h, t: dict, m: dict, eps: float, stored=exact) -> torch.Tensor:
    """Half the sum of the two mixers' outputs, each RMS-normed over the model width first."""
    left = windowed_mixer(h, sub(t, "left."), m["left"], eps, stored)
    right = delta_mixer(h, sub(t, "right."), m["right"], eps, stored)
    return 0.5 * (rms_norm(left, t["left.out"], eps) + rms_norm(right, t["right.out"], eps))


# ----------------------------------------------------------------------------- the model
def sub(tensors: dict, prefix: str) -> dict:
    return {name[len(prefix):]: value for name, value in tensors.items() if name.startswith(prefix)}


def feed_forward(h, t: dict, stored=exact) -> torch.Tensor:
    return stored(stored(gelu_tanh(stored(h @ t["gate"].T)) * stored(h @ t["up"].T)) @ t["down"].T)


def forward(config: dict, tensors: dict, tokens: list[int], stored=exact):
    """(logits [n, vocab], the stream after every layer [layers, n, W]) of one whole sequence. `tensors`
    by name, as stored; `config` is the parsed config.json."""
    tensors = {name: value.to(F) for name, value in tensors.items()}
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    n = len(tokens)
    x = tensors["embed"][tokens] + tensors["pos"][:n]
    streams, latents = [], {}
    for index, layer in enumerate(config["layers"]):
        t, m = sub(tensors, f"l{index}."), layer["mixer"]
        h = stored(x)
        if layer["type"] == "latent_attention":
            source = m.get("kv_from")
            mixed, made = latent_mixer(h, sub(t, "mix."), m, eps, stored, None if source is None else latents[source])
            latents[index] = made
        elif layer["type"] == "parallel":
            mixed = side_by_side_mixer(h, sub(t, "mix."), m, eps, stored)
        else:
            raise ValueError(layer["type"])
        x = rms_norm(alpha * x + mixed, t["norm1"], eps)
        if layer.get("mlp"):
            x = rms_norm(alpha * x + feed_forward(stored(x), sub(t, "mlp."), stored), t["norm2"], eps)
        streams.append(x)
    logits = stored(rms_norm(x, tensors["final.norm"], eps)) @ tensors["head"].T
    return logits, torch.stack(streams)
