"""A plain, slow implementation of the Pedorax decoder, one function per mechanism, written
from the design's equations in float64.  It is the oracle of the tests: it shares no code
with the package, processes a whole sequence at once (the recurrent mixer token by token)
and keeps no cache.

Notation: ``h`` is a [T, width] block of normalised rows, ``W`` matrices are stored
[out, in] and applied as ``h @ W.T``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def prepare(raw, round_to=None):
    """float64 copies of the stored tensors (integer tables stay integers); ``round_to``
    rounds matrices to that type first, as a model bound for it holds them."""
    out = {}
    for name, t in raw.items():
        if not t.dtype.is_floating_point:
            out[name] = t.clone()
            continue
        if round_to is not None and t.dim() >= 2:
            t = t.to(round_to)
        out[name] = t.to(F64)
    return out


# ---------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------

def dynamic_tanh(x, weight, bias, alpha):
    """tanh(alpha x) * weight + bias, elementwise: no statistic of the row enters."""
    return torch.tanh(alpha * x) * weight + bias


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_pairs(v, positions, base, dims):
    """Rotary positions, interleaved: the pair (2i, 2i+1) of the first ``dims`` entries turns
    by the angle position * base^(-2i/dims); the rest pass unchanged.  v [T, ..., n]."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)      # [half]
    ang = positions.to(F64).view(-1, *([1] * (v.dim() - 1))) * freq               # [T, .., half]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------------------------------
# latent attention
# ---------------------------------------------------------------------------------------

def latent_keys(h, w, pre, m, eps):
    """What a latent-attention layer caches per token: the normed latent [T, kv_rank] and the
    shared rotated key part [T, rot_dim] (after rotation)."""
    R, P = m["kv_rank"], m["rot_dim"]
    T = h.shape[0]
    d = h @ w[pre + "dkv"].T
    c = rms_unit(d[:, :R], eps) * w[pre + "dkv.norm"]
    kr = rotate_pairs(d[:, R:R + P], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, w, pre, m, c, kr):
    """Causal attention whose keys and values are expanded from a shared latent; the softmax's
    denominator also holds exp(sink) per head."""
    H, D, P, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, D + P)
    q_plain = q[:, :, :D]
    q_rot = rotate_pairs(q[:, :, D:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[pre + "uk"].T).view(T, H, D)
    val = (c @ w[pre + "uv"].T).view(T, H, V)
    sink = w[pre + "sink"]
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ kr.T) * m["scale"]     # [T, T]
        for i in range(T):
            row = s[i, :i + 1]
            top = max(float(row.max()), float(sink[hd]))
            e = torch.exp(row - top)
            den = e.sum() + math.exp(float(sink[hd]) - top)
            out[i, hd] = (e / den) @ val[:i + 1, hd]
    return out.reshape(T, H * V) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------
# gated delta rule with a decay per key channel
# ---------------------------------------------------------------------------------------

def short_conv(x, taps_w):
    """Causal convolution over time per channel: taps_w [C, taps], last column weighs the
    current token, zeros before the start.  x [T, C]."""
    T, C = x.shape
    n = taps_w.shape[1]
    pad = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x])
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + pad[j:j + T] * taps_w[:, j]
    return y


def channel_delta(h, w, pre, m, eps):
    H, HK, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).view(T, HK, D)
    k = silu(short_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).view(T, HK, D)
    v = silu(short_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                       # [T, H]
    step = softplus((h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(w[pre + "A_log"]).view(1, H, 1) * step)           # [T, H, D]
    gate = torch.sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, V)
    rep = H // HK
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=F64)
        kh = hd // rep
        for t in range(T):
            S = decay[t, hd].view(D, 1) * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, hd] = S.T @ q[t, kh]
    out = rms_unit(out, eps) * w[pre + "norm"] * gate
    return out.reshape(T, H * V) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------------
# routed feed-forward
# ---------------------------------------------------------------------------------------

def route(z, r):
    """Expert choice of one token from its router logits z [E]: (indices, weights)."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(z)
    n_groups, keep = r["groups"]["count"], r["groups"]["keep"]
    per = E // n_groups
    g = s.view(n_groups, per)
    g_score = torch.topk(g, min(2, per), dim=-1).values.sum(-1)
    allowed_groups = torch.topk(g_score, keep).indices
    mask = torch.zeros(n_groups, per, dtype=torch.bool)
    mask[allowed_groups] = True
    masked = torch.where(mask.view(E), s, torch.full_like(s, -1.0))
    idx = torch.topk(masked, top).indices
    wt = s[idx]
    return idx, wt / (wt.sum() + 1e-20)


def expert(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def routed_feed_forward(h, w, pre, f):
    T = h.shape[0]
    z = h @ w[pre + "router"].T
    out = torch.zeros(T, w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(T):
        idx, wt = route(z[t], f["router"])
        for e, a in zip(idx.tolist(), wt):
            out[t] += a * expert(h[t:t + 1], w, f"{pre}e{e}.", f["expert"]["limit"])[0]
    return out


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (float64); with ``return_layers`` also the
    residual stream after every layer [layers, T, width]."""
    tok = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tok] * cfg["embedding"]["scale"]
    kept = {}
    trail = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = dynamic_tanh(x, w[p + "norm1"], w[p + "norm1.b"], w[p + "norm1.alpha"])
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_keys(h, w, p + "mix.", m, eps)
                src = i
            y = latent_attention(h, w, p + "mix.", m, *kept[src])
        elif layer["type"] == "channel_delta":
            y = channel_delta(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            y = y + routed_feed_forward(h, w, p + "mlp.", layer["mlp"])
        x = x + y
        trail.append(x.clone())
    hf = dynamic_tanh(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"])
    logits = (hf @ w["embed"].T) * cfg["logit_scale"]
    if return_layers:
        return logits, torch.stack(trail)
    return logits
