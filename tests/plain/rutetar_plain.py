"""Plain, slow forward pass of the Rutetar design: whole sequences, no cache, CPU only.

One function per mechanism, written from the design's equations, computing with torch on
the CPU in float64 (or float32).  It shares no code with the product package: it reads
config.json with json and the weights with the `safetensors` library.

Notation: X is the residual stream as `streams` copies [S, T, width]; h is what a sublayer reads
[T, width]; t is a token's index in its sequence (its position, from 0); W is a weight stored
[out, in] and applied as W h.
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


# -- norms --------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Over the last axis: x / sqrt(mean(x^2) + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The design's norm: the stored weight lies around zero, the gain is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# -- hyper-connections ----------------------------------------------------------------------------
def streams_read(X: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """u = sum_s in[s] X[s]."""
    return torch.einsum("s,std->td", w_in, X)


def streams_write(X: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """All streams at once from the old ones: X'[t] = sum_s mix[s, t] X[s] + out[t] y."""
    return torch.einsum("sr,std->rtd", mix, X) + w_out[:, None, None] * y[None]


# -- rotary positions --------------------------------------------------------------------------
def rotate(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, heads, d]: of each head's first `dims` entries, entry i and entry i + dims/2 are a pair (a, b) that becomes
    (a cos - b sin, b cos + a sin) with the angle position * base^(-2i/dims); the other entries stay."""
    half = dims // 2
    if half == 0:
        return v
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(ang).to(v.dtype)[:, None, :], torch.sin(ang).to(v.dtype)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


# -- the softmax attention with a window, biases and a gate per head ------------------------------
def window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query head h reads key/value head h // (H/G); token t sees
    the tokens j with 0 <= t - j < window."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            lo = max(0, t - window + 1)
            s = (k[lo:t + 1, g] @ q[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[lo:t + 1, g]
    return out


def gated_window_mixer(h: torch.Tensor, w: dict, p: str, m: dict, positions: torch.Tensor) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q, k = rotate(q, positions, rot["dims"], rot["base"]), rotate(k, positions, rot["dims"], rot["base"])
    window = m["mask"]["size"] if m.get("mask") else T       # without a mask: every token before
    o = window_attention(q, k, v, m["scale"], window)
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * dv) @ w[p + "o"].T


# -- the time-mixing recurrence with a decay per token and channel --------------------------------
def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """h + (h' - h) * mu with h' the row before (zeros in front of the first)."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu


def bonus_recurrence(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """r, k, v, decay [T, H, d], u [H, d] -> o [T, H, d]:  o_t = (S + diag(u) k_t v_t^T)^T r_t, then S = diag(decay_t) S + k_t v_t^T."""
    T, H, d = r.shape
    out = torch.zeros_like(v)
    for hd in range(H):
        S = torch.zeros((d, d), dtype=r.dtype)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = decay[t, hd][:, None] * S + kv
    return out


def time_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    mix = {s: token_shift(h, w[p + "mu." + s]) for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, d)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, d)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, d)
    gate = silu(mix["g"] @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    o = bonus_recurrence(r, k, v, decay, w[p + "u"].view(H, d))
    o = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    left = gated_window_mixer(h, w, p + "left.", m["left"], positions)
    right = time_mixer(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# -- retention: a fixed decay per head, no softmax -------------------------------------------------
def fixed_decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: list) -> torch.Tensor:
    """q, k [T, H, d], v [T, H, dv] -> o [T, H, dv]:  S = decay_h S + k_t v_t^T, then o_t = S^T q_t."""
    T, H, d = q.shape
    out = torch.zeros_like(v)
    for hd in range(H):
        S = torch.zeros((d, v.shape[-1]), dtype=q.dtype)
        for t in range(T):
            S = float(decay[hd]) * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    return out


def retention_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, H, d) * d ** -0.5
    v = (h @ w[p + "v"].T).view(T, H, dv)
    o = unit_rms(fixed_decay_recurrence(q, k, v, m["decay"]), eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


# -- feed-forwards --------------------------------------------------------------------------------
def gated_feed_forward(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act) -> torch.Tensor:
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, bias: torch.Tensor, top: int):
    """The `top` largest router outputs (ties: lower index) and the softmax over those alone."""
    z = h @ router.T + bias
    order = sorted(range(z.shape[0]), key=lambda e: (-float(z[e]), e))[:top]
    zs = torch.stack([z[e] for e in order])
    return order, torch.softmax(zs, dim=0)


def mixture(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weight = route(h[t], w[p + "router"], w[p + "router.b"], top)
        for e, g in zip(chosen, weight):
            q = f"{p}e{e}."
            out[t] += g * gated_feed_forward(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"], silu)[0]
    return out


def feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_feed_forward(h, w[p + "gate"], w[p + "up"], w[p + "down"], gelu_tanh)
    return mixture(h, w, p, mlp)


# -- the model ---------------------------------------------------------------------------------
def layer_order(config: dict) -> list:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config: dict, w: dict, tokens: list, layers_out: bool = False):
    """Logits [T, vocab] of one sequence (and, asked for, the sum of the streams after every layer run)."""
    eps = config["norm"]["eps"]
    dtype = w["embed"].dtype
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)]
    S = config.get("streams")
    X = torch.stack([x] * (S or 1))
    seen = []
    for i in layer_order(config):
        layer, p = config["layers"][i], f"l{i}."
        for q, sub in ((1, "mixer"), (2, "mlp")):
            if sub == "mlp" and layer.get("mlp") is None:
                continue
            if S:
                u = streams_read(X, w[f"{p}hc{q}.in"])
            else:
                u = X[0]
            h = offset_norm(u, w[f"{p}norm{q}"], eps)
            if sub == "mlp":
                y = feed_forward(h, w, p + "mlp.", layer["mlp"])
            elif layer["type"] == "retention":
                y = retention_mixer(h, w, p + "mix.", layer["mixer"], eps)
            elif layer["type"] == "parallel":
                y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, positions)
            else:
                raise ValueError(layer["type"])
            if S:
                X = streams_write(X, y, w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"])
            else:
                X = X + y[None]
        seen.append(X.sum(0))
    x = offset_norm(X.sum(0), w["final.norm"], eps)
    logits = (x @ w["head"].T).to(dtype)
    return (logits, torch.stack(seen)) if layers_out else logits


def greedy(config: dict, weights: dict, prompt, new_tokens: int) -> list:
    tokens, out = list(prompt), []
    for _ in range(new_tokens):
        nxt = int(torch.argmax(forward(config, weights, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
