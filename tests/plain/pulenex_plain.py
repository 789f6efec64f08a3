"""Plain, slow forward pass of the Pulenex design: whole sequences, no cache, CPU only.

One function per mechanism, written from the design's equations, computing with torch on
the CPU in float64 (or float32).  It shares no code with the product package: it reads
config.json with json and the weights with the `safetensors` library.

Notation: x is the residual stream [T, width]; h is what a sublayer reads [T, width]; t is a
token's index in its sequence (its position, from 0); W is a weight stored [out, in] and applied
as W h.
"""
from __future__ import annotations

import json
import math
import os

import torch


def read_model(folder: str, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return config, weights


# -- norms and activations ------------------------------------------------------------------------
def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(variance + eps) * w over the last axis; the variance is the mean squared deviation."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# -- rotary positions -------------------------------------------------------------------------------
def _angles(positions: torch.Tensor, dims: int, base: float):
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    return torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, heads, d]: of each head's first `dims` entries, entries i and i + dims/2 are a pair (a, b) -> (a cos - b sin, b cos + a sin)."""
    if dims == 0:
        return v
    half = dims // 2
    c, s = (z.to(v.dtype) for z in _angles(positions, dims, base))
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """The same with entries 2i and 2i + 1 as the pairs."""
    if dims == 0:
        return v
    c, s = (z.to(v.dtype) for z in _angles(positions, dims, base))
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    turned = torch.stack([a * c - b * s, b * c + a * s], dim=-1).reshape(*v.shape[:-1], dims)
    return torch.cat([turned, v[..., dims:]], dim=-1)


# -- a short causal convolution over time ---------------------------------------------------------------
def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros in front of the sequence."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


# -- retention -------------------------------------------------------------------------------------
def retention(h, W, p, m, eps, positions):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half(q, positions, rot["dims"], rot["base"])
    k = rotate_half(k, positions, rot["dims"], rot["base"]) * d ** -0.5
    o = torch.zeros((T, H, dv), dtype=h.dtype)
    for a in range(H):
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(T):
            S = m["decay"][a] * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# -- the left of a parallel layer: chunked softmax attention whose heads talk ---------------------------------------
def talking_attention(h, W, p, m, positions):
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = short_conv(h @ W[p + "q"].T, W[p + "q.conv"]).reshape(T, H, d)
    k = short_conv(h @ W[p + "k"].T, W[p + "k.conv"]).reshape(T, G, d)
    v = k                                                   # the values are the keys before the rotation
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_pairs(q, positions, rot["dims"], rot["base"])
    kr = rotate_pairs(k, positions, rot["dims"], rot["base"])
    rep = H // G
    s = torch.stack([q[:, a] @ kr[:, a // rep].T for a in range(H)]) * m["scale"] * W[p + "temp"][:, None, None]   # [H, T, T]
    s = torch.einsum("hg,gij->hij", W[p + "talk"], s)
    size = m["mask"]["size"] if m.get("mask") else None
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if size:
        seen = seen & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    s = s.masked_fill(~seen[None], float("-inf"))
    sink = W[p + "sink"][:, None, None]
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    w = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
    o = torch.stack([w[a] @ v[:, a // rep] for a in range(H)], dim=1).reshape(T, H * d)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# -- the right of a parallel layer: the gated delta rule ----------------------------------------------------------
def gated_delta(h, W, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                            # [T, H]
    step = softplus((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).reshape(T, H, d)
    decay = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * step)               # [T, H, d]
    rep = H // G
    o = torch.zeros((T, H, dv), dtype=h.dtype)
    for a in range(H):
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(T):
            kt, qt = k[t, a // rep], q[t, a // rep]
            S = decay[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ kt)
            S = S + torch.outer(kt, u)
            o[t, a] = S.T @ qt
    o = unit_rms(o, eps) * W[p + "norm"]
    o = o.reshape(T, H * dv) * torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T)
    return o @ W[p + "o"].T


def parallel(h, W, p, m, eps, positions):
    left = talking_attention(h, W, p + "left.", m["left"], positions)
    right = gated_delta(h, W, p + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * W[p + "left.out"] + unit_rms(right, eps) * W[p + "right.out"])


# -- latent attention ---------------------------------------------------------------------------------
def latent_rows(h, W, p, m, eps, positions):
    """What a layer caches: the normed latent c [T, kv_rank] and the rotated key part [T, rot_dim]."""
    r = m["kv_rank"]
    row = h @ W[p + "dkv"].T
    c = unit_rms(row[:, :r], eps) * W[p + "dkv.norm"]
    kr = rotate_pairs(row[:, None, r:], positions, m["rot_dim"], m["rot"]["base"])[:, 0]
    return c, kr


def latent_attention(h, W, p, m, positions, c, kr):
    T = h.shape[0]
    H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d + dr)
    qn, qr = q[..., :d], rotate_pairs(q[..., d:], positions, dr, m["rot"]["base"])
    kn = (c @ W[p + "uk"].T).reshape(T, H, d)
    v = (c @ W[p + "uv"].T).reshape(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if m.get("mask"):
        seen = seen & (i - j < m["mask"]["size"])
    s = s.masked_fill(~seen[None], float("-inf"))
    w = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", w, v) * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


# -- feed-forward ---------------------------------------------------------------------------------------
def clamped_glu(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T + W[p + "gate.b"], max=limit)
    u = torch.clamp(h @ W[p + "up"].T + W[p + "up.b"], min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T + W[p + "down.b"]


# -- the model ----------------------------------------------------------------------------------------
def forward(config: dict, W: dict, tokens, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = W["embed"][tokens]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "retention":
            y = retention(h, W, p + "mix.", m, eps, positions)
        elif layer["type"] == "parallel":
            y = parallel(h, W, p + "mix.", m, eps, positions)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_rows(h, W, p + "mix.", m, eps, positions)
            c, kr = kept[i if m.get("kv_from") is None else m["kv_from"]]
            y = latent_attention(h, W, p + "mix.", m, positions, c, kr)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, W[p + "norm2"], eps)
            x = x + layer_norm(clamped_glu(h, W, p + "mlp.", layer["mlp"]["limit"]), W[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (layer_norm(x, W["final.norm"], eps) @ W["head"].T) * config.get("logit_scale", 1.0)


def greedy(config: dict, W: dict, prompt, n: int) -> list:
    """n tokens, each the argmax of the logits behind everything before it (the lowest index among equals)."""
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(forward(config, W, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
